// tcgen05 tensor-core panels of the fused linear + cross-entropy head.
//
// One persistent GEMM kernel, D[M,N] (+)= A[M,K] . B[N,K]^T, each operand read from memory either
// K-major ([MN][K], K contiguous) or MN-major ([K][MN], MN contiguous):
//   warp 0      : TMA producer  - cp.async.bulk.tensor tiles (128-byte swizzle) into a ring of
//                 shared-memory stages, completion on mbarriers;
//   warp 1      : allocates TMEM, then one elected lane issues tcgen05.mma (M = 128, N = BN with
//                 cta_group::1; M = 256 over a pair of CTAs with cta_group::2) from shared-memory
//                 descriptors into one of two TMEM accumulators; tcgen05.commit releases stages and
//                 publishes accumulators;
//   warps 2..9  : epilogue - tcgen05.ld of the finished accumulator (one TMEM lane = one output
//                 row per thread), store / accumulate to global memory, while the MMA warp
//                 already works on the next tile in the other accumulator.
// Precision modes:
//   3xTF32 : every fp32 operand is split once into hi = tf32(x), lo = tf32(x - hi); each k-step
//            issues hi*lo + lo*hi + hi*hi into the same fp32 accumulator (error ~2^-22 of the
//            product, i.e. fp32-grade logits from tf32 tensor cores);
//   BF16   : operands rounded to bf16 once, a single MMA per k-step.
//   BF16X3 : every fp32 operand is split once into hi = bf16(x), lo = bf16(x - hi); the same three
//            MMAs per k-step at the bf16 rate on half the operand bytes (error ~2^-17 of the
//            product: measured like 3xTF32 on the gradients, 3e-5 to 5e-5 of their rms, and 1e-7 on the
//            loss; not good enough for a per-element forward output held to 1e-5).
// The three GEMMs of the head read X, W and dl as stored; no transposed copy exists:
//   logits  = X   . W^T       A = X  [rows,C] K-major     B = W [vc,C]   K-major
//   dX     += dl  . W         A = dl [rows,vc] K-major    B = W [vc,C]   MN-major (contraction over vc)
//   dW     += dl^T. X         A = dl [rows,vc] MN-major   B = X [rows,C] MN-major (contraction over rows)
// An MN-major tile is fetched as one 3-d TMA box {128 bytes of MN, BK k-rows, MN groups} (one 2-d box per
// group when the MN extent is ragged) and described to the MMA with the transposing descriptor forms
// (see TcDesc).
// Every output tile has exactly one writer, so accumulation order is fixed.
// Every mbarrier wait is bounded; on expiry the CTA raises AG_STATUS_WAIT_EXPIRED, all roles
// leave their loops, TMEM is released and the kernel returns.  The split-operand modes run on clusters
// of two CTAs (see tc_gemm_kernel); every CTA loads its own tiles with plain (single-destination) TMA
// loads.
// Accumulation inside the tensor core truncates, so the length of an accumulation chain is bounded by
// split-K where a workspace exists (see tc_gemm).
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
  int a_mn, b_mn;  // operand is MN-major in memory ([K][MN], MN contiguous) instead of K-major ([MN][K])
  int mn_group;    // MN elements per 128-byte row of an MN-major tile (32 fp32 / 64 bf16)
  int a_3d, b_3d;  // MN-major operand fetched as one 3-d box {MN group, BK, groups} instead of one box per group
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
  void* dl_hi;             // EPI_DLOGITS output: dl [M][ld_dl], (hi, lo) or bf16
  void* dl_lo;
  int64_t ld_dl;
};

enum { EPI_STORE = 0, EPI_STATS = 1, EPI_DLOGITS = 2 };
// operand modes (AgTcMode of ag_flce.cuh): tf32 (hi, lo) pairs, bf16 values, bf16 (hi, lo) pairs
enum { TC_TF32X3 = AG_TC_TF32X3, TC_BF16 = AG_TC_BF16, TC_BF16X3 = AG_TC_BF16X3 };
constexpr bool tc_mode_tf32(int mode) { return mode == TC_TF32X3; }
constexpr bool tc_mode_split(int mode) { return mode != TC_BF16; }

// ---------------------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ void tc_tma_load_2d(const CUtensorMap* tm, void* smem_dst, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          ag_smem_u32(smem_dst)),
      "l"(tm), "r"(ag_smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

__device__ __forceinline__ void tc_tma_load_3d(const CUtensorMap* tm, void* smem_dst, uint64_t* bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(
          ag_smem_u32(smem_dst)),
      "l"(tm), "r"(ag_smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(ag_smem_u32(bar))
               : "memory");
}

// One MMA from the two halves of each shared-memory descriptor (low word: address and leading byte
// offset, high word: stride byte offset, version, layout).  ACC = 2: accumulate flag from a register
// (the first MMA of a stage), ACC = 1: always accumulate (no predicate set-up instruction).
// PAIR: the instruction spans a pair of CTAs (cta_group::2, M = 256): issued by the leader CTA only,
// it reads A rows and B columns from the shared memory of both CTAs at the same offsets and writes
// 128 accumulator rows into the tensor memory of each.
#define TC_MMA_ASM(GROUP, KIND, SETP)                                                              \
  "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t" SETP "\n\t"                                     \
  "mov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"                                           \
  "tcgen05.mma.cta_group::" GROUP ".kind::" KIND " [%0], da, db, %5, p;\n\t}"
template <bool TF32, int ACC, bool PAIR>
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi,
                                       uint32_t idesc, uint32_t accumulate) {
#define TC_MMA_CASE(GROUP, KIND)                                                                                 \
  if (ACC == 2)                                                                                                  \
    asm volatile(TC_MMA_ASM(GROUP, KIND, "setp.ne.b32 p, %6, 0;")::"r"(tmem_d), "r"(a_lo), "r"(a_hi), "r"(b_lo), \
                 "r"(b_hi), "r"(idesc), "r"(accumulate)                                                          \
                 : "memory");                                                                                    \
  else                                                                                                           \
    asm volatile(TC_MMA_ASM(GROUP, KIND, "setp.eq.b32 p, 0, 0;")::"r"(tmem_d), "r"(a_lo), "r"(a_hi), "r"(b_lo),  \
                 "r"(b_hi), "r"(idesc)                                                                           \
                 : "memory");
  if (TF32) {
    if (PAIR) { TC_MMA_CASE("2", "tf32") } else { TC_MMA_CASE("1", "tf32") }
  } else {
    if (PAIR) { TC_MMA_CASE("2", "f16") } else { TC_MMA_CASE("1", "f16") }
  }
#undef TC_MMA_CASE
}

// ---- CTA pair (thread-block cluster of 2) helpers
__device__ __forceinline__ uint32_t tc_cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t tc_map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void tc_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// commit whose mbarrier may live in either CTA of the pair
__device__ __forceinline__ void tc_commit_pair(uint32_t cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr) : "memory");
}
// tile loads of a CTA of the pair: destination in the own shared memory, completion bytes counted on
// the mbarrier at `mbar_cluster_addr`, which is the leader's
__device__ __forceinline__ void tc_tma_load_2d_pair(const CUtensorMap* tm, void* smem_dst, uint32_t mbar_cluster_addr,
                                                    int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::
          "r"(ag_smem_u32(smem_dst)),
      "l"(tm), "r"(mbar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tc_tma_load_3d_pair(const CUtensorMap* tm, void* smem_dst, uint32_t mbar_cluster_addr,
                                                    int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], "
      "[%2];" ::"r"(ag_smem_u32(smem_dst)),
      "l"(tm), "r"(mbar_cluster_addr), "r"(x), "r"(y), "r"(z)
      : "memory");
}

// Shared-memory matrix descriptors (version 1, Blackwell), as two 32-bit words.
//   low word : bits 0-13 start address >> 4, bits 16-29 leading byte offset >> 4
//   high word: bits 0-13 stride byte offset >> 4, bit 14 version, bits 29-31 layout type
// K-major operand, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart (stride byte
// offset 64), leading byte offset unused (1), layout 2; one MMA consumes 32 bytes of K inside the row,
// so consecutive MMAs advance the start address by 2 units.
// MN-major operand: the tile is stored as [MN group][k row][128 bytes of MN]; consecutive MN groups
// are BK * 128 bytes apart (leading byte offset).  16-bit operands use the plain 128-byte swizzle,
// whose atom is 8 k rows (stride byte offset 64, layout 2).  32-bit operands can only be transposed
// by the tensor core from the 128-byte swizzle with 32-byte atomicity (layout 1): its atom is 4 k rows
// (stride byte offset 32), and the matching TMA mode swizzles 32-byte chunks by the row index modulo
// 4.  One MMA consumes umma_k k-rows of 128 bytes: 64 (tf32) or 128 (bf16) address units.
template <bool TF32>
struct TcDesc {
  uint32_t lo_const, hi, step;
  __device__ __forceinline__ void init(int mn_major, uint32_t group_bytes) {
    if (mn_major) {
      lo_const = ((group_bytes >> 4) & 0x3FFFu) << 16;
      hi = TF32 ? (32u | (1u << 14) | (1u << 29)) : (64u | (1u << 14) | (2u << 29));
      step = TF32 ? 64u : 128u;
    } else {
      lo_const = 1u << 16;
      hi = 64u | (1u << 14) | (2u << 29);
      step = 2u;
    }
  }
};

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

// 32-byte (whole sector) global accesses of one lane: the epilogues give every lane 128 contiguous
// bytes of its own row, which four of these cover with full-sector writes (16-byte stores fill half a
// sector per request).  Addresses must be 32-byte aligned.
struct F8 { float v[8]; };
__device__ __forceinline__ F8 tc_ld_global_v8(const float* p) {
  F8 r;
  asm volatile("ld.global.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=f"(r.v[0]), "=f"(r.v[1]), "=f"(r.v[2]), "=f"(r.v[3]), "=f"(r.v[4]), "=f"(r.v[5]), "=f"(r.v[6]), "=f"(r.v[7])
               : "l"(p));
  return r;
}
__device__ __forceinline__ void tc_st_global_v8(float* p, const float* v) {
  asm volatile("st.global.v8.f32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]),
               "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7])
               : "memory");
}
__device__ __forceinline__ void tc_st_global_v8_b32(void* p, const uint32_t* v) {
  asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]),
               "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
               : "memory");
}

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

// PAIR: launched as clusters of two CTAs that share every 256-row output tile (see tc_mma): CTA `rank`
// owns rows [128 rank, 128 rank + 128) of the tile and loads its own A rows and half of the B columns,
// so a pair pulls a third less operand data through shared memory than two single CTAs.  All stage
// barriers that the MMA waits on live in the leader (rank 0); the leader's commits arrive on the
// barriers of both CTAs.
template <int MODE, int EPI, bool PAIR>
__global__ void __launch_bounds__(TC_THREADS, 1)
tc_gemm_kernel(const __grid_constant__ CUtensorMap tmA_hi, const __grid_constant__ CUtensorMap tmA_lo,
               const __grid_constant__ CUtensorMap tmB_hi, const __grid_constant__ CUtensorMap tmB_lo,
               const TcParams p) {
  constexpr bool TF32 = tc_mode_tf32(MODE);    // element type of the operands: tf32 (in fp32 words) or bf16
  constexpr bool SPLIT = tc_mode_split(MODE);  // operands come as (hi, lo) pairs, three MMAs per k-step
  extern __shared__ unsigned char tc_smem_raw[];
  // tiles need 1024-byte alignment for the 128-byte swizzle pattern
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(tc_smem_raw) + 1023) & ~(uintptr_t)1023);
  const uint32_t stage_bytes = (p.a_bytes + p.b_bytes) * (SPLIT ? 2u : 1u);
  uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + (size_t)p.stages * stage_bytes);
  uint64_t* full = bars;
  uint64_t* empty = bars + TC_MAX_STAGES;
  uint64_t* acc_full = bars + 2 * TC_MAX_STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = PAIR ? tc_cluster_rank() : 0u;
  // this CTA's (pair's) position in the stream of output tiles, and the stream's stride
  const int unit = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int unit_stride = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  const int row_off = PAIR ? (int)rank * TC_BM : 0;        // first row of this CTA inside the tile
  const int bm_tile = PAIR ? 2 * TC_BM : TC_BM;            // rows of an output tile
  const int bn_cta = PAIR ? p.BN / 2 : p.BN;               // B columns this CTA loads

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      ag_mbar_init(&full[s], 1);
      ag_mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      ag_mbar_init(&acc_full[b], 1);
      ag_mbar_init(&acc_empty[b], PAIR ? 16 : 8);  // one arrival per epilogue warp (of both CTAs)
    }
    *abort_flag = 0;
    if (PAIR)
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    else
      ag_fence_mbar_init();
  }
  if (PAIR) tc_cluster_sync(); else __syncthreads();  // the peer's barriers exist before anything arrives on them
  if (warp == 1) {
    // 512 columns: two accumulators of up to 256 fp32 columns each (this kernel owns the SM)
    if (PAIR) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(ag_smem_u32(tmem_slot)),
                   "r"(512u)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(ag_smem_u32(tmem_slot)),
                   "r"(512u)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int total_tiles = p.tiles_m * p.tiles_n * p.splits;
  bool expired = false;
  // Everything above touched no global memory and may overlap the tail of the previous kernel of the
  // stream; from here on its results are read.  The grid is a single wave, so the next kernel may be
  // scheduled as soon as this one's CTAs leave their SMs.
  ag_pdl_wait();
  ag_pdl_trigger();

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      for (int tile = unit; tile < total_tiles && !expired; tile += unit_stride) {
        int tm, tn, k_begin, k_end, split_id;
        tc_tile_coords(p, tile, tm, tn, k_begin, k_end, split_id);
        const int m0 = tm * bm_tile + row_off, n0 = tn * p.BN + (PAIR ? (int)rank * bn_cta : 0);
        for (int k = k_begin; k < k_end; ++k) {
          if (!tc_wait(&empty[stage], phase ^ 1u, abort_flag)) {
            expired = true;
            break;
          }
          unsigned char* s = tiles + (size_t)stage * stage_bytes;
          // pair: the leader's barrier counts the bytes of both CTAs' loads; a completion that arrives
          // before the leader has posted its expectation only makes the pending count negative for a while
          uint32_t full_addr = ag_smem_u32(&full[stage]);
          if (PAIR) {
            if (rank == 0) ag_mbar_expect_tx(&full[stage], 2u * stage_bytes);
            full_addr = tc_map_to_cta(full_addr, 0u);
          } else {
            ag_mbar_expect_tx(&full[stage], stage_bytes);
          }
          const int kx = k * p.BK;
          // K-major operand: one box {BK, rows}.  MN-major operand: one box {128 bytes of MN, BK rows} per
          // MN group, stored group after group.
          const uint32_t gbytes = (uint32_t)p.BK * 128u;
          auto load_operand = [&](const CUtensorMap* tm, unsigned char* dst, int mn0, int mn_rows, int mn_major, int is3d) {
            if (PAIR) {
              if (!mn_major) {
                tc_tma_load_2d_pair(tm, dst, full_addr, kx, mn0);
              } else if (is3d) {
                tc_tma_load_3d_pair(tm, dst, full_addr, 0, kx, mn0 / p.mn_group);
              } else {
                for (int g = 0; g * p.mn_group < mn_rows; ++g)
                  tc_tma_load_2d_pair(tm, dst + (size_t)g * gbytes, full_addr, mn0 + g * p.mn_group, kx);
              }
            } else if (!mn_major) {
              tc_tma_load_2d(tm, dst, &full[stage], kx, mn0);
            } else if (is3d) {
              tc_tma_load_3d(tm, dst, &full[stage], 0, kx, mn0 / p.mn_group);
            } else {
              for (int g = 0; g * p.mn_group < mn_rows; ++g)
                tc_tma_load_2d(tm, dst + (size_t)g * gbytes, &full[stage], mn0 + g * p.mn_group, kx);
            }
          };
          load_operand(&tmA_hi, s, m0, TC_BM, p.a_mn, p.a_3d);
          if (SPLIT) {
            load_operand(&tmA_lo, s + p.a_bytes, m0, TC_BM, p.a_mn, p.a_3d);
            load_operand(&tmB_hi, s + 2 * p.a_bytes, n0, bn_cta, p.b_mn, p.b_3d);
            load_operand(&tmB_lo, s + 2 * p.a_bytes + p.b_bytes, n0, bn_cta, p.b_mn, p.b_3d);
          } else {
            load_operand(&tmB_hi, s + p.a_bytes, n0, bn_cta, p.b_mn, p.b_3d);
          }
          if (++stage == (uint32_t)p.stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (pair: the leader only)
    if (lane == 0 && rank == 0) {
      uint32_t stage = 0, phase = 0;
      uint32_t acc_par[2] = {0, 0};
      int local = 0;
      // Everything an MMA needs beyond two additions is prepared outside the k loop: this one thread
      // issues 12 (3xTF32) or 4 (bf16) MMAs per stage and its instruction stream is on the critical path.
      TcDesc<TF32> dA, dB;
      dA.init(p.a_mn, (uint32_t)p.BK * 128u);
      dB.init(p.b_mn, (uint32_t)p.BK * 128u);
      const uint32_t a_lo_off = p.a_bytes >> 4, b_lo_off = p.b_bytes >> 4;
      const uint32_t b_off = (SPLIT ? 2u * p.a_bytes : p.a_bytes) >> 4;
      const uint32_t stage_units = stage_bytes >> 4;
      const uint32_t tiles_u = ag_smem_u32(tiles) >> 4;
      for (int tile = unit; tile < total_tiles && !expired; tile += unit_stride, ++local) {
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
          const uint32_t su = tiles_u + stage * stage_units;
          const uint32_t ah = su + dA.lo_const, al = ah + a_lo_off;   // A hi / lo tiles
          const uint32_t bh = su + b_off + dB.lo_const, bl = bh + b_lo_off;
          const uint32_t not_first = (k != k_begin) ? 1u : 0u;
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {  // BK / umma_k = 4 MMAs along K per stage in both modes
            const uint32_t ao = (uint32_t)kk * dA.step, bo = (uint32_t)kk * dB.step;
            if (SPLIT) {
              if (kk == 0)
                tc_mma<TF32, 2, PAIR>(tacc, ah + ao, dA.hi, bl + bo, dB.hi, p.idesc, not_first);
              else
                tc_mma<TF32, 1, PAIR>(tacc, ah + ao, dA.hi, bl + bo, dB.hi, p.idesc, 1u);
              tc_mma<TF32, 1, PAIR>(tacc, al + ao, dA.hi, bh + bo, dB.hi, p.idesc, 1u);
              tc_mma<TF32, 1, PAIR>(tacc, ah + ao, dA.hi, bh + bo, dB.hi, p.idesc, 1u);
            } else {
              if (kk == 0)
                tc_mma<TF32, 2, PAIR>(tacc, ah + ao, dA.hi, bh + bo, dB.hi, p.idesc, not_first);
              else
                tc_mma<TF32, 1, PAIR>(tacc, ah + ao, dA.hi, bh + bo, dB.hi, p.idesc, 1u);
            }
          }
          // stage reusable once these MMAs have read it (pair: in both CTAs)
          if (PAIR) {
            const uint32_t e = ag_smem_u32(&empty[stage]);
            tc_commit_pair(tc_map_to_cta(e, 0u));
            tc_commit_pair(tc_map_to_cta(e, 1u));
          } else {
            tc_commit(&empty[stage]);
          }
          if (++stage == (uint32_t)p.stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (expired) break;
        // accumulator complete (pair: each CTA's epilogue waits on its own barrier)
        if (PAIR) {
          const uint32_t f = ag_smem_u32(&acc_full[buf]);
          tc_commit_pair(tc_map_to_cta(f, 0u));
          tc_commit_pair(tc_map_to_cta(f, 1u));
        } else {
          tc_commit(&acc_full[buf]);
        }
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
    // 32-byte accesses: rows and bases aligned to a sector
    const bool vec_ok = ((p.ldd & 7) == 0) && ((reinterpret_cast<uintptr_t>(p.D) & 31u) == 0) &&
                        (!p.bias || (reinterpret_cast<uintptr_t>(p.bias) & 31u) == 0) &&
                        (!p.resid || (((p.ld_resid & 7) == 0) && (reinterpret_cast<uintptr_t>(p.resid) & 31u) == 0));
    for (int tile = unit; tile < total_tiles; tile += unit_stride, ++local) {
      const int buf = local & 1;
      int tm, tn, k_begin, k_end, split_id;
      tc_tile_coords(p, tile, tm, tn, k_begin, k_end, split_id);
      const int m0 = tm * bm_tile + row_off, n0 = tn * p.BN;
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
              // all loads of a source are issued before anything is stored: with a load and a store per
              // packet in one loop the eight round trips to memory would be taken one after the other
              float* dst = drow + col;
              float v[32];
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
              if (p.accumulate) {
                F8 o[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) o[j] = tc_ld_global_v8(dst + 8 * j);
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] += o[j >> 3].v[j & 7];
              }
              if (p.bias) {
                F8 o[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) o[j] = tc_ld_global_v8(p.bias + col + 8 * j);
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] += o[j >> 3].v[j & 7];
              }
              if (p.resid) {
                const float* rsrc = p.resid + (int64_t)row * p.ld_resid + col;
                F8 o[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) o[j] = tc_ld_global_v8(rsrc + 8 * j);
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] += o[j >> 3].v[j & 7];
              }
#pragma unroll
              for (int j = 0; j < 4; ++j) tc_st_global_v8(dst + 8 * j, v + 8 * j);
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
        // dlogits of this row, written in operand form (hi, lo) or bf16
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
        // 32-byte stores: whole-sector rows (8 floats, 16 bf16) on sector-aligned bases
        const bool row_vec = ((p.ld_dl & 15) == 0) && ((reinterpret_cast<uintptr_t>(p.dl_hi) & 31u) == 0) &&
                             (!p.dl_lo || (reinterpret_cast<uintptr_t>(p.dl_lo) & 31u) == 0);
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
            } else if (SPLIT) {
              hi[j] = __bfloat162float(__float2bfloat16_rn(d));  // stored as bf16 below without further rounding
              lo[j] = d - hi[j];
            } else {
              hi[j] = d;
            }
          }
          if (TF32) {
            float* dh = static_cast<float*>(p.dl_hi) + (int64_t)row * p.ld_dl + col;
            float* dlo = static_cast<float*>(p.dl_lo) + (int64_t)row * p.ld_dl + col;
            if (row_vec && col + 32 <= p.N) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                tc_st_global_v8(dh + j, hi + j);
                tc_st_global_v8(dlo + j, lo + j);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col + j < p.N) { dh[j] = hi[j]; dlo[j] = lo[j]; }
            }
          } else {
            // bf16 operands: the values, or for the split mode the (hi, lo) pair of bf16 arrays
            auto store_bf16 = [&](void* base, const float (&val)[32]) {
              __nv_bfloat16* dh = static_cast<__nv_bfloat16*>(base) + (int64_t)row * p.ld_dl + col;
              if (row_vec && col + 32 <= p.N) {
#pragma unroll
                for (int j = 0; j < 32; j += 16) {
                  uint32_t w[8];
#pragma unroll
                  for (int q2 = 0; q2 < 8; ++q2) {
                    __nv_bfloat162 h2 = __floats2bfloat162_rn(val[j + 2 * q2], val[j + 2 * q2 + 1]);
                    w[q2] = *reinterpret_cast<uint32_t*>(&h2);
                  }
                  tc_st_global_v8_b32(dh + j, w);
                }
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (col + j < p.N) dh[j] = __float2bfloat16_rn(val[j]);
              }
            };
            store_bf16(p.dl_hi, hi);
            if (SPLIT) store_bf16(p.dl_lo, lo);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (PAIR)
          tc_mbar_arrive_cluster(tc_map_to_cta(ag_smem_u32(&acc_empty[buf]), 0u));  // the leader's MMA thread waits
        else
          ag_mbar_arrive(&acc_empty[buf]);
      }
    }
  }
  if (expired && lane == 0) atomicOr(p.status, AG_STATUS_WAIT_EXPIRED);
  tc_fence_before();
  // pair: neither CTA may leave, or free its tensor memory, while the other can still read its shared
  // memory or arrive on its barriers
  if (PAIR) tc_cluster_sync(); else __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    if (PAIR)
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    else
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

// ---------------------------------------------------------------------------- host side
struct TcOperand {
  const void* hi;
  const void* lo;   // null in bf16 mode
  int64_t ld;       // elements between consecutive rows of the array as stored
  int mn_major;     // 0: stored [MN][K] (K contiguous); 1: stored [K][MN] (MN contiguous)
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
              int box_k, int box_rows, bool atom32 = false) {
  EncodeTiledFn encode = tc_encode_fn(ctx);
  if (!encode) return AG_ERR_CUDA;
  const size_t es = bf16 ? 2 : 4;
  cuuint64_t dims[2] = {(cuuint64_t)k_extent, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * es};
  cuuint32_t box[2] = {(cuuint32_t)box_k, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = encode(tm, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2,
                                      const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                      atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    AG_FAIL(ctx, AG_ERR_CUDA, "cuTensorMapEncodeTiled failed: CUresult %d (ptr %p, k %lld, rows %lld, ld %lld, box %dx%d)",
            (int)r, ptr, (long long)k_extent, (long long)rows, (long long)ld, box_k, box_rows);
  return AG_OK;
}

// MN-major operand stored [K][mn_extent] (row stride ld) seen as {group elements, K, groups}: one box
// {group, box_k, box_groups} lands in shared memory as [group][k row][128 bytes].
int tc_encode_mn3(ag_ctx* ctx, CUtensorMap* tm, const void* ptr, bool bf16, int64_t mn_extent, int64_t k_extent,
                  int64_t ld, int group, int box_k, int box_groups) {
  EncodeTiledFn encode = tc_encode_fn(ctx);
  if (!encode) return AG_ERR_CUDA;
  const size_t es = bf16 ? 2 : 4;
  cuuint64_t dims[3] = {(cuuint64_t)group, (cuuint64_t)k_extent, (cuuint64_t)(mn_extent / group)};
  cuuint64_t strides[2] = {(cuuint64_t)ld * es, (cuuint64_t)group * es};
  cuuint32_t box[3] = {(cuuint32_t)group, (cuuint32_t)box_k, (cuuint32_t)box_groups};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = encode(tm, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3,
                      const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                      bf16 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B,
                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    AG_FAIL(ctx, AG_ERR_CUDA, "cuTensorMapEncodeTiled (3-d) failed: CUresult %d (ptr %p, mn %lld, k %lld, ld %lld)", (int)r,
            ptr, (long long)mn_extent, (long long)k_extent, (long long)ld);
  return AG_OK;
}

// D[m][n] (+)= sum over splits, in split order, of the partial outputs P[s][m][n].
// VEC: N, ldd multiples of 4 and 16-byte aligned pointers: one 16-byte packet per thread and split,
// all splits' packets requested before the first add.
template <bool VEC>
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(const float* __restrict__ P, int splits, int M, int N, float* D, int64_t ldd, int accumulate) {
  ag_pdl_wait();
  const int64_t total = (int64_t)M * N;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  if (VEC) {
    const int n4 = N >> 2;
    const int64_t packets = (int64_t)M * n4;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < packets; i += stride) {
      const int m = (int)(i / n4), n = (int)(i - (int64_t)m * n4) << 2;
      float4* d = reinterpret_cast<float4*>(D + (int64_t)m * ldd + n);
      const float* src = P + (int64_t)m * N + n;
      float4 acc = accumulate ? *d : make_float4(0.f, 0.f, 0.f, 0.f);
      int sp = 0;
      for (; sp + 4 <= splits; sp += 4) {
        float4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) v[u] = __ldcs(reinterpret_cast<const float4*>(src + (int64_t)(sp + u) * total));
#pragma unroll
        for (int u = 0; u < 4; ++u) { acc.x += v[u].x; acc.y += v[u].y; acc.z += v[u].z; acc.w += v[u].w; }
      }
      for (; sp < splits; ++sp) {
        const float4 v = __ldcs(reinterpret_cast<const float4*>(src + (int64_t)sp * total));
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
      *d = acc;
    }
  } else {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
      const int m = (int)(i / N), n = (int)(i - (int64_t)m * N);
      float* d = D + (int64_t)m * ldd + n;
      float acc = accumulate ? *d : 0.0f;
      for (int sp = 0; sp < splits; ++sp) acc += P[(int64_t)sp * total + i];
      *d = acc;
    }
  }
}

// Largest number of CTA pairs (clusters of 2) of this kernel that are resident at once; 0 on error.
template <int MODE, int EPI>
int tc_max_pairs(ag_ctx* ctx, size_t smem) {
  static int cached_dev[AG_MAX_DEVICES];
  static size_t cached_smem_dev[AG_MAX_DEVICES];
  static bool init_done = false;
  if (!init_done) {
    for (int i = 0; i < AG_MAX_DEVICES; ++i) cached_dev[i] = -1;
    init_done = true;
  }
  int& cached = cached_dev[ag_dev_slot(ctx)];
  size_t& cached_smem = cached_smem_dev[ag_dev_slot(ctx)];
  if (cached >= 0 && cached_smem == smem) return cached;
  auto kern = tc_gemm_kernel<MODE, EPI, true>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM_LIMIT) != cudaSuccess) return 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * ctx->sm_count);
  cfg.blockDim = dim3(TC_THREADS);
  cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = 2;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) {
    cudaGetLastError();
    n = 0;
  }
  cached = n;
  cached_smem = smem;
  return n;
}

template <int MODE, int EPI, bool PAIR>
int tc_launch(ag_ctx* ctx, int grid, size_t smem, const CUtensorMap& a_hi, const CUtensorMap& a_lo,
              const CUtensorMap& b_hi, const CUtensorMap& b_lo, const TcParams& p) {
  static bool attr_done[AG_MAX_DEVICES] = {};
  auto kern = tc_gemm_kernel<MODE, EPI, PAIR>;
  if (!attr_done[ag_dev_slot(ctx)]) {
    AG_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM_LIMIT));
    attr_done[ag_dev_slot(ctx)] = true;
  }
  int rc_ev;
  if (ctx->tc_timing && (rc_ev = ag_event_record(ctx, ctx->tc_timing_base + 2 * ctx->tc_timing_count))) return rc_ev;
  {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(TC_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute at[2];
    int n_at = 0;
    if (PAIR) {
      at[n_at].id = cudaLaunchAttributeClusterDimension;
      at[n_at].val.clusterDim.x = 2;
      at[n_at].val.clusterDim.y = 1;
      at[n_at].val.clusterDim.z = 1;
      ++n_at;
    }
    if (ctx->pdl) {
      at[n_at].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      at[n_at].val.programmaticStreamSerializationAllowed = 1;
      ++n_at;
    }
    cfg.attrs = at;
    cfg.numAttrs = n_at;
    AG_CUDA(ctx, cudaLaunchKernelEx(&cfg, kern, a_hi, a_lo, b_hi, b_lo, p));
    ctx->launches++;
  }
  if (ctx->tc_timing) {
    if ((rc_ev = ag_event_record(ctx, ctx->tc_timing_base + 2 * ctx->tc_timing_count + 1))) return rc_ev;
    ctx->tc_timing_count++;
  }
  return AG_OK;
}

template <int EPI>
int tc_launch_any(ag_ctx* ctx, int mode, bool pair, int grid, size_t smem, const CUtensorMap& a_hi,
                  const CUtensorMap& a_lo, const CUtensorMap& b_hi, const CUtensorMap& b_lo, const TcParams& p) {
#define TC_LAUNCH_MODE(M)                                                                      \
  return pair ? tc_launch<M, EPI, true>(ctx, grid, smem, a_hi, a_lo, b_hi, b_lo, p)            \
              : tc_launch<M, EPI, false>(ctx, grid, smem, a_hi, a_lo, b_hi, b_lo, p);
  switch (mode) {
    case TC_TF32X3: TC_LAUNCH_MODE(TC_TF32X3)
    case TC_BF16: TC_LAUNCH_MODE(TC_BF16)
    default: TC_LAUNCH_MODE(TC_BF16X3)
  }
#undef TC_LAUNCH_MODE
}

// `epi` (may be null = EPI_STORE) carries the fields of the fused cross-entropy epilogues.
int tc_gemm(ag_ctx* ctx, int mode, const TcOperand& A, const TcOperand& B, float* D, int64_t ldd, int M, int N, int K,
            bool accumulate, int epi_kind = EPI_STORE, const TcParams* epi = nullptr, int* tiles_n_out = nullptr,
            float* splitk_ws = nullptr, size_t splitk_ws_bytes = 0) {
  TcParams p = {};
  if (epi) p = *epi;
  p.M = M; p.N = N; p.K = K;
  const bool bf16 = !tc_mode_tf32(mode);  // element type of the operands
  p.BK = bf16 ? 64 : 32;
  p.umma_k = bf16 ? 16 : 8;
  p.split = tc_mode_split(mode) ? 1 : 0;
  // Tile width, split-K factor and CTA pairing.  Measured behaviour of this kernel: a k-step costs
  // time in proportion to the operand bytes a CTA pulls through shared memory (128 A rows + the B rows
  // it loads: BN, or BN/2 as one CTA of a pair), a tile costs about 8 k-steps of prologue / epilogue on
  // top, and CTAs (pairs) work in rounds over the SMs (SM pairs).  Split-K is only considered for
  // plain accumulate outputs with a workspace and few tiles.
  const int cand[] = {256, 192, 160, 128};
  int best_bn = 128, best_s = 1, best_pair = 0;
  double best_cost = 1e300;
  const int k_iters_all = (K + p.BK - 1) / p.BK;
  p.a_mn = A.mn_major ? 1 : 0;
  p.b_mn = B.mn_major ? 1 : 0;
  p.mn_group = bf16 ? 64 : 32;
  // CTA pairs: measured faster for 3xTF32 (0.56-0.67 ms against 0.61-0.75 ms per 16384 x 4096 x 1280
  // panel) and no gain for plain bf16, whose stages are half as large: pairs are used by the split
  // modes.  AG_B200_TC_PAIR=0 keeps single CTAs.
  int n_pairs = 0;
  if (p.split && M > TC_BM && ctx->tc_pair)
    n_pairs = bf16 ? tc_max_pairs<TC_BF16X3, EPI_STORE>(ctx, 200 * 1024) : tc_max_pairs<TC_TF32X3, EPI_STORE>(ctx, 200 * 1024);
  for (int pair = 0; pair <= (n_pairs > 0 ? 1 : 0); ++pair) {
    const int units = pair ? n_pairs : ctx->sm_count;
    const int tiles_m_c = (M + (pair ? 2 : 1) * TC_BM - 1) / ((pair ? 2 : 1) * TC_BM);
    for (int bn : cand) {
      const int bn_cta = pair ? bn / 2 : bn;
      if (p.b_mn && bn_cta % p.mn_group != 0) continue;
      if (pair && bn % 32 != 0) continue;
      const int tn = (N + bn - 1) / bn;
      const int64_t tiles = (int64_t)tiles_m_c * tn;
      // Split-K serves two purposes.  Speed: few tiles are spread over more CTAs.  Accuracy: the tensor
      // core adds every MMA into the fp32 accumulator with truncation, a bias that grows with the length
      // of the accumulation chain (measured on dW, 16384 rows: 2.7e-4 of the rms with one chain, 3.6e-5
      // with 8, for tf32; bf16 MMAs about three times that); the partial sums of the splits are added
      // with round-to-nearest.  So K per chain is bounded whenever a workspace allows it.
      int s_max = 1, s_min = 1;
      if (epi_kind == EPI_STORE && splitk_ws) {
        const int64_t fit = (int64_t)(splitk_ws_bytes / ((size_t)M * N * sizeof(float)));
        const int k_chain = bf16 ? 1024 : 2048;  // contraction elements per accumulation chain
        s_min = (K + k_chain - 1) / k_chain;
        if (s_min > 16) s_min = 16;
        if (s_min > fit) s_min = fit < 1 ? 1 : (int)fit;
        if (tiles < 2 * (int64_t)units) {
          s_max = k_iters_all / 16;
          if (s_max > 16) s_max = 16;
          if (s_max > fit) s_max = (int)fit;
        }
        if (s_max < s_min) s_max = s_min;
        if (s_max < 1) s_max = 1;
        if (p.split == 0) s_min = 1;  // plain bf16 (2e-2): no accuracy constraint
      }
      for (int sp = s_min; sp <= s_max; ++sp) {
        const int k_per = (k_iters_all + sp - 1) / sp;
        const int s_eff = (k_iters_all + k_per - 1) / k_per;
        const int64_t rounds = (tiles * s_eff + units - 1) / units;
        // (a pair works on half as many, twice as tall tiles with half as many units: same rounds)
        double cost = (double)rounds * (k_per + 8) * (128 + bn_cta);
        if (s_eff > 1) cost += 0.02 * cost;  // the ordered reduction of the partial outputs
        if (cost < best_cost) {
          best_cost = cost;
          best_bn = bn;
          best_s = s_eff;
          best_pair = pair;
        }
      }
    }
  }
  const bool pair = best_pair != 0;
  const int bm_tile = pair ? 2 * TC_BM : TC_BM;
  const int tiles_m = (M + bm_tile - 1) / bm_tile;
  const int units = pair ? n_pairs : ctx->sm_count;
  p.BN = best_bn;
  const int bn_cta = pair ? p.BN / 2 : p.BN;
  p.tiles_m = tiles_m;
  p.tiles_n = (N + p.BN - 1) / p.BN;
  if (tiles_n_out) *tiles_n_out = p.tiles_n;
  p.k_iters = k_iters_all;
  p.k_per_split = (p.k_iters + best_s - 1) / best_s;
  p.splits = (p.k_iters + p.k_per_split - 1) / p.k_per_split;
  p.split_stride = 0;
  p.a_bytes = (uint32_t)TC_BM * 128u;
  p.b_bytes = (uint32_t)bn_cta * 128u;
  const uint32_t stage_bytes = (p.a_bytes + p.b_bytes) * (p.split ? 2u : 1u);
  int stages = (TC_SMEM_LIMIT - 1024 - 256) / (int)stage_bytes;
  if (stages > TC_MAX_STAGES) stages = TC_MAX_STAGES;
  AG_REQUIRE(ctx, stages >= 2, "tc_gemm: tile does not fit shared memory");
  p.stages = stages;
  // per-wave operand footprint decides the tile order (keep the re-read operand in L2)
  {
    const int64_t sm = units;
    const int64_t ab = (int64_t)p.a_bytes * (pair ? 2 : 1), bb = (int64_t)p.b_bytes * (pair ? 2 : 1);
    const int64_t fp_m_fast = (tiles_m < sm ? tiles_m : sm) * ab + ((sm + tiles_m - 1) / tiles_m) * bb;
    const int64_t fp_n_fast = (p.tiles_n < sm ? p.tiles_n : sm) * bb + ((sm + p.tiles_n - 1) / p.tiles_n) * ab;
    p.n_fastest = fp_n_fast <= fp_m_fast ? 1 : 0;
  }
  // instruction descriptor: D fp32, A/B tf32 or bf16, operand majors, N>>3 at bit 17, M>>4 at bit 24
  // (M = 256 for the instruction that spans a CTA pair)
  const uint32_t fmt = bf16 ? 1u : 2u;
  p.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)p.a_mn << 15) | ((uint32_t)p.b_mn << 16) |
            ((uint32_t)(p.BN >> 3) << 17) | ((uint32_t)(bm_tile >> 4) << 24);
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
  // tensor maps: K-major {K inner, MN rows} with box {BK, tile rows}; MN-major {MN inner, K rows} with
  // box {one 128-byte MN group, BK}
  // whole MN groups: one 3-d box per operand tile; a ragged MN extent falls back to one 2-d box per group
  p.a_3d = (p.a_mn && M % p.mn_group == 0) ? 1 : 0;
  p.b_3d = (p.b_mn && N % p.mn_group == 0) ? 1 : 0;
  auto encode_operand = [&](CUtensorMap* tm, const void* ptr, const TcOperand& op, int mn_extent, int tile_rows) -> int {
    if (!op.mn_major) return tc_encode(ctx, tm, ptr, bf16, K, mn_extent, op.ld, p.BK, tile_rows);
    if (mn_extent % p.mn_group == 0)
      return tc_encode_mn3(ctx, tm, ptr, bf16, mn_extent, K, op.ld, p.mn_group, p.BK, tile_rows / p.mn_group);
    return tc_encode(ctx, tm, ptr, bf16, mn_extent, K, op.ld, p.mn_group, p.BK, /*atom32=*/!bf16);
  };
  if ((rc = encode_operand(&tA_hi, A.hi, A, M, TC_BM))) return rc;
  if ((rc = encode_operand(&tB_hi, B.hi, B, N, bn_cta))) return rc;
  if (p.split) {
    if ((rc = encode_operand(&tA_lo, A.lo, A, M, TC_BM))) return rc;
    if ((rc = encode_operand(&tB_lo, B.lo, B, N, bn_cta))) return rc;
  } else {
    tA_lo = tA_hi;
    tB_lo = tB_hi;
  }
  const size_t smem = 1024 + (size_t)stages * stage_bytes + 256;
  const int64_t total = (int64_t)p.tiles_m * p.tiles_n * p.splits;
  const int grid = (int)(total < units ? total : units) * (pair ? 2 : 1);
  if (epi_kind == EPI_STATS) {
    AG_REQUIRE(ctx, p.part_ld >= M, "tc_gemm: partial-statistics rows too short");
    return tc_launch_any<EPI_STATS>(ctx, mode, pair, grid, smem, tA_hi, tA_lo, tB_hi, tB_lo, p);
  }
  if (epi_kind == EPI_DLOGITS) return tc_launch_any<EPI_DLOGITS>(ctx, mode, pair, grid, smem, tA_hi, tA_lo, tB_hi, tB_lo, p);
  rc = tc_launch_any<EPI_STORE>(ctx, mode, pair, grid, smem, tA_hi, tA_lo, tB_hi, tB_lo, p);
  if (rc || p.splits == 1) return rc;
  const int64_t n4 = ((int64_t)M * N + 3) / 4;
  int64_t want = (n4 + 255) / 256;
  if (want > (int64_t)ctx->sm_count * 8) want = (int64_t)ctx->sm_count * 8;
  const bool vec = (N % 4 == 0) && (ldd % 4 == 0) && ((reinterpret_cast<uintptr_t>(D) & 15u) == 0) &&
                   ((reinterpret_cast<uintptr_t>(splitk_ws) & 15u) == 0);
  if (vec)
    AG_LAUNCH_PDL(ctx, "splitk_reduce_kernel", splitk_reduce_kernel<true>, (int)want, 256, 0, (const float*)splitk_ws,
                  p.splits, M, N, D, ldd, accumulate ? 1 : 0);
  else
    AG_LAUNCH_PDL(ctx, "splitk_reduce_kernel", splitk_reduce_kernel<false>, (int)want, 256, 0, (const float*)splitk_ws,
                  p.splits, M, N, D, ldd, accumulate ? 1 : 0);
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

// src[R][Cc] (row stride lds) -> operand form [R][Cc] (row stride ldo): (hi, lo) tf32 pairs, or bf16
// values in `hi`.  Cc, lds and ldo are multiples of 4; one thread converts 4 consecutive elements.
template <int MODE>
__global__ void __launch_bounds__(256)
split_kernel(const float* __restrict__ src, int64_t lds, void* __restrict__ hi, void* __restrict__ lo, int64_t ldo,
             int R, int Cc) {
  const int c4 = Cc >> 2;
  const int64_t total = (int64_t)R * c4;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t r = i / c4;
    const int c = (int)(i - r * c4) << 2;
    const float4 x = *reinterpret_cast<const float4*>(src + r * lds + c);
    if (MODE == TC_TF32X3) {
      float4 h, l;
      split_tf32(x.x, h.x, l.x);
      split_tf32(x.y, h.y, l.y);
      split_tf32(x.z, h.z, l.z);
      split_tf32(x.w, h.w, l.w);
      *reinterpret_cast<float4*>(static_cast<float*>(hi) + r * ldo + c) = h;
      *reinterpret_cast<float4*>(static_cast<float*>(lo) + r * ldo + c) = l;
    } else {
      __nv_bfloat162 a = __floats2bfloat162_rn(x.x, x.y), b = __floats2bfloat162_rn(x.z, x.w);
      *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(hi) + r * ldo + c) =
          make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b));
      if (MODE == TC_BF16X3) {  // lo = bf16(x - hi)
        const float2 fa = __bfloat1622float2(a), fb = __bfloat1622float2(b);
        __nv_bfloat162 la = __floats2bfloat162_rn(x.x - fa.x, x.y - fa.y), lb = __floats2bfloat162_rn(x.z - fb.x, x.w - fb.y);
        *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(lo) + r * ldo + c) =
            make_uint2(*reinterpret_cast<uint32_t*>(&la), *reinterpret_cast<uint32_t*>(&lb));
      }
    }
  }
}

// Folds the per-tile (max, sum exp) partials of one panel into the running row statistics, tiles
// in index order (fixed order, one thread per row).
__global__ void __launch_bounds__(256)
ce_merge_partials_kernel(const float2* __restrict__ part, int64_t part_ld, int tiles_n, int rows,
                         float* __restrict__ run_max, float* __restrict__ run_sum, int first_panel) {
  ag_pdl_wait();
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
inline int tc_mode_of(int precision) {
  return precision == AG_CE_BF16 ? TC_BF16 : (precision == AG_CE_BF16X3 ? TC_BF16X3 : TC_TF32X3);
}

struct TcPlan {
  int64_t rows_tile, vc;
  size_t es;  // operand element size
  size_t X_hi, X_lo, W_hi, W_lo, dl_hi, dl_lo, part, splitk, splitk_bytes, total;
  int64_t part_ld;
};

inline size_t up256(size_t x) { return (x + 255) & ~(size_t)255; }
inline int64_t up8(int64_t x) { return (x + 7) & ~(int64_t)7; }
inline int64_t up16(int64_t x) { return (x + 15) & ~(int64_t)15; }  // dl rows: whole 32-byte sectors in bf16 too

TcPlan tc_plan(const ag_flce_desc* d) {
  TcPlan p;
  const int mode = tc_mode_of(d->precision);
  const bool bf16 = mode == TC_BF16;  // one array per operand (no lo part)
  p.es = tc_mode_tf32(mode) ? 4 : 2;
  p.rows_tile = d->N < AG_FLCE_ROWS_TILE ? d->N : AG_FLCE_ROWS_TILE;
  p.vc = d->vocab_chunk < d->V ? d->vocab_chunk : d->V;
  const int64_t ldr = up8(p.rows_tile), ldc = up16(p.vc);
  size_t off = 0;
  auto take = [&](size_t elems) { size_t o = off; off += up256(elems * p.es); return o; };
  p.X_hi = take((size_t)d->N * d->C);
  p.X_lo = bf16 ? p.X_hi : take((size_t)d->N * d->C);
  p.W_hi = take((size_t)d->V * d->C);
  p.W_lo = bf16 ? p.W_hi : take((size_t)d->V * d->C);
  p.dl_hi = take((size_t)p.rows_tile * ldc);
  p.dl_lo = bf16 ? p.dl_hi : take((size_t)p.rows_tile * ldc);
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

int tc_split(ag_ctx* ctx, int mode, const float* src, int64_t lds, void* hi, void* lo, int64_t ldo, int64_t R, int Cc) {
  AG_REQUIRE(ctx, Cc % 4 == 0 && lds % 4 == 0 && ldo % 4 == 0 && R < (1ll << 31), "tc_split: rows must be whole 16-byte packets");
  int64_t want = (R * (Cc / 4) + 255) / 256;
  if (want > (int64_t)ctx->sm_count * 16) want = (int64_t)ctx->sm_count * 16;
  if (want < 1) want = 1;
  if (mode == TC_TF32X3)
    split_kernel<TC_TF32X3><<<(int)want, 256, 0, ctx->stream>>>(src, lds, hi, lo, ldo, (int)R, Cc);
  else if (mode == TC_BF16)
    split_kernel<TC_BF16><<<(int)want, 256, 0, ctx->stream>>>(src, lds, hi, lo, ldo, (int)R, Cc);
  else
    split_kernel<TC_BF16X3><<<(int)want, 256, 0, ctx->stream>>>(src, lds, hi, lo, ldo, (int)R, Cc);
  AG_LAUNCHED(ctx, "split_kernel");
  return AG_OK;
}

}  // namespace

// ---- entry points for other translation units (ag_flce.cuh) ---------------------------------
int ag_tc_gemm(ag_ctx* ctx, int mode, const AgTcOperand& A, const AgTcOperand& B, float* D, int64_t ldd, int M, int N,
               int K, bool accumulate, const float* bias, const float* resid, int64_t ld_resid, float* splitk_ws,
               size_t splitk_ws_bytes) {
  TcParams e = {};
  e.bias = bias;
  e.resid = resid;
  e.ld_resid = ld_resid;
  TcOperand a{A.hi, A.lo, A.ld, A.mn_major}, b{B.hi, B.lo, B.ld, B.mn_major};
  return tc_gemm(ctx, mode, a, b, D, ldd, M, N, K, accumulate, EPI_STORE, &e, nullptr, splitk_ws, splitk_ws_bytes);
}

int ag_tc_split(ag_ctx* ctx, int mode, const float* src, int64_t lds, void* hi, void* lo, int64_t ldo, int64_t R,
                int Cc) {
  return tc_split(ctx, mode, src, lds, hi, lo, ldo, R, Cc);
}

// =========================================================================================
bool ag_flce_tc_supported(const ag_flce_desc* d) {
  if (d->precision != AG_CE_3XTF32 && d->precision != AG_CE_BF16 && d->precision != AG_CE_BF16X3) return false;
  // TMA needs 16-byte aligned row starts: rows of X / W are C elements long
  const int q = d->precision == AG_CE_3XTF32 ? 4 : 8;
  if (d->C % q != 0) return false;
  if (d->vocab_chunk % 8 != 0 && d->vocab_chunk < d->V) return false;
  if (d->C < 32 || d->V < 32 || d->N < 1) return false;
  return true;
}

size_t ag_flce_tc_scratch_bytes(const ag_flce_desc* d) { return tc_plan(d).total; }

int ag_flce_tc_prepare(ag_ctx* ctx, const ag_flce_desc* d, const float* X, const float* W, void* tc_scratch) {
  const TcPlan p = tc_plan(d);
  unsigned char* b = static_cast<unsigned char*>(tc_scratch);
  const int mode = tc_mode_of(d->precision);
  int rc;
  if ((rc = tc_split(ctx, mode, X, d->C, b + p.X_hi, b + p.X_lo, d->C, d->N, d->C))) return rc;
  return tc_split(ctx, mode, W, d->C, b + p.W_hi, b + p.W_lo, d->C, d->V, d->C);
}

int ag_flce_tc_forward_panel(ag_ctx* ctx, const ag_flce_desc* d, void* tc_scratch, int64_t r0, int rows, int v0,
                             int vc, const int32_t* targets, float* run_max, float* run_sum, float* tgt_logit,
                             bool first_panel) {
  const TcPlan p = tc_plan(d);
  unsigned char* b = static_cast<unsigned char*>(tc_scratch);
  const int mode = tc_mode_of(d->precision);
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
  int rc = tc_gemm(ctx, mode, A, B, nullptr, 0, rows, vc, d->C, false, EPI_STATS, &e, &tiles_n);
  if (rc) return rc;
  AG_LAUNCH_PDL(ctx, "ce_merge_partials_kernel", ce_merge_partials_kernel, (rows + 255) / 256, 256, 0,
                (const float2*)e.part, e.part_ld, tiles_n * 2, rows, run_max + r0, run_sum + r0, first_panel ? 1 : 0);
  return AG_OK;
}

int ag_flce_tc_grads(ag_ctx* ctx, const ag_flce_desc* d, void* tc_scratch, int64_t r0, int rows, int v0, int vc,
                     const int32_t* targets, const float* lse, const float* row_scale, const float* dloss,
                     const float* denom, float* dX, float* dW) {
  const TcPlan p = tc_plan(d);
  unsigned char* b = static_cast<unsigned char*>(tc_scratch);
  const int mode = tc_mode_of(d->precision);
  const int64_t ldc = up16(p.vc);
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
    if ((rc = tc_gemm(ctx, mode, A, B, nullptr, 0, rows, vc, d->C, false, EPI_DLOGITS, &e))) return rc;
  }
  if (dX) {
    // dX[r0:r0+rows, :] += dl [rows, vc] . W[v0:v0+vc, :]; W as stored has the contraction index
    // (vocabulary) as its row index, i.e. it is the MN-major form of the B operand.  Panels wider than
    // 4096 are taken in pieces of 4096 columns: bounded accumulation chains (see tc_gemm), the pieces
    // are added by the accumulating epilogue.
    for (int k0 = 0; k0 < vc; k0 += 4096) {
      const int kc = vc - k0 < 4096 ? vc - k0 : 4096;
      TcOperand A{b + p.dl_hi + (size_t)k0 * p.es, b + p.dl_lo + (size_t)k0 * p.es, ldc, 0};
      TcOperand B{b + p.W_hi + (size_t)(v0 + k0) * row_bytes, b + p.W_lo + (size_t)(v0 + k0) * row_bytes, d->C, 1};
      if ((rc = tc_gemm(ctx, mode, A, B, dX + r0 * d->C, d->C, rows, d->C, kc, true))) return rc;
    }
  }
  if (dW) {
    // dW[v0:v0+vc, :] += dl^T . X[r0:r0+rows, :]; the contraction index (row) is the row index of
    // both dl and X as stored: both operands MN-major
    TcOperand A{b + p.dl_hi, b + p.dl_lo, ldc, 1};
    TcOperand B{b + p.X_hi + (size_t)r0 * row_bytes, b + p.X_lo + (size_t)r0 * row_bytes, d->C, 1};
    if ((rc = tc_gemm(ctx, mode, A, B, dW + (int64_t)v0 * d->C, d->C, vc, d->C, rows, true, EPI_STORE, nullptr, nullptr,
                      reinterpret_cast<float*>(b + p.splitk), p.splitk_bytes)))
      return rc;
  }
  return AG_OK;
}
