// Prefill GEMM  y[M, N] = x[M, K] . W[N, K]^T (+ bias)  for the mixed-precision layer,
// sm_100a: dequantise-to-shared-memory producers feeding tcgen05 kind::f16 MMAs with the
// FP32 accumulator in tensor memory.
//
// Tile: 128 or 256 tokens x 128 or 256 output channels per CTA (chosen per launch by a time
// estimate, see gemm_plan), k blocks of 64.  The output tile is taken in ORIGINAL channel order:
// channel n0 + j reads permuted row inv_perm[n0 + j], so the permutation costs nothing on the
// store side (rows of all three formats meet in one tile).
//
//   warp 0 (1 thread)   TMA (cp.async.bulk.tensor.2d, 128B swizzle) loads of the 128 x 64
//                       activation blocks into the A stage (one per 128 tokens).
//   warp 1 (1 thread)   issues 4 x tcgen05.mma (M128, N = tile width, K16) per k block and
//                       128-token accumulator, commits the stage back to the producers,
//                       finally commits the accumulators.  The warp also owns the
//                       tensor-memory allocation (up to all 512 columns).
//   warps 2..           12 or 22 dequantisation warps.  The rows of the tile are sorted by
//                       format and padded to groups of four; a warp takes every W-th group,
//                       a quarter warp one row, a lane one 16-byte chunk (8 k) of it: it
//                       loads the next k block's 4 / 8 / 16 packed bytes into registers,
//                       converts the current ones to f16 (NVFP4: hardware E2M1 converter
//                       times the block scale, exact in f16; FP8: E4M3 converter, channel
//                       scale deferred to the epilogue; FP16: copy) and stores its chunk in
//                       the K-major 128B-swizzled layout the MMA descriptor expects -- the
//                       eight lanes of a row write 128 contiguous bytes (no bank conflicts)
//                       and read 32 / 64 / 128 contiguous bytes.
//   epilogue            twelve of those warps: tcgen05.ld of the accumulators (a warp reads
//                       the 32 tensor-memory lanes of its quarter, the warps of a quarter
//                       take pairs of 32-column chunks in turn), channel scale and bias, f16
//                       conversion, transposition through the free stage buffers, stores of
//                       4 rows x 128 contiguous bytes per instruction.
//
// Shared memory: 4 stages x (16 or 32 KB A + 16 KB B), or 3 x (32 KB A + 32 KB B) for the
// 256 x 256 tile.  All mbarrier waits are bounded; a wait that runs out raises an abort flag
// that every role checks, and the kernel drains and frees its tensor memory.
//
// Measured on B200 (in-kernel clocks, 256 x 256 tile): with the weight conversion switched
// off the pipeline runs at the MMA rate (1024 cycles per k block); with it, about 1450 cycles.
// Shared-memory bandwidth is the bound: per k block the MMAs read 96 KB (A and B once per
// M128 instruction), TMA writes 32 KB and the producers 32 KB = 160 KB at 128 B/clk.
//
// FLOPs per launch: 2*M*N*K.  Bound: dense f16 tensor throughput.
//
// Reference behaviour replaced: F.linear over a materialised FP16 weight copy
// (rdquant/inference.py:679-687) and 2 x marlin_gemm + F.linear + cat + index_select
// (rdquant/inference.py:620-677).
#include <cuda.h>

#include "rdq_kernels.cuh"

namespace rdq {

namespace {

constexpr int BM = 128, BK = 64;
constexpr int kStageA = BM * BK * 2;  // 16 KB: one 128-token activation block
constexpr int kMaxBN = 256;

// Tile configurations.  BN = output channels per CTA (= N of one tcgen05.mma), MT = 128-token
// accumulators per CTA.  Producer warps convert groups of four weight rows (a quarter warp per
// row); kTasks = groups a warp handles per k block.
//   <1,128> <2,128>: 12 producer warps, 4 stages         (small problems)
//   <2,256>        : 22 producer warps (768 threads), 3 x 64 KB stages, all 512 tensor-memory columns
template <int MT, int BN>
struct GemmCfg {
  static constexpr int kProducerWarps = (BN == 128) ? 12 : 22;
  static constexpr int kProducers = kProducerWarps * 32;
  static constexpr int kThreads = (2 + kProducerWarps) * 32;
  static constexpr int kStageB = BN * BK * 2;
  static constexpr int kStageAll = kStageA * MT;
  static constexpr int kStages = (BN == 128) ? 4 : 3;
  static constexpr int kTmemCols = BN * MT;  // power of two >= 32
  static constexpr int kSmem = kStages * (kStageAll + kStageB) + 1024;
  static constexpr int kMaxQuads = BN / 4 + 3;  // each format padded to a multiple of four rows
  static constexpr int kTasks = (kMaxQuads + kProducerWarps - 1) / kProducerWarps;
  static constexpr int kPrefetch = 1;  // k blocks of packed weights held in registers ahead of use
};

struct GemmSmem {
  // dynamic part starts 1024-byte aligned: A stages, then B stages
  // static part:
  uint64_t full[4];
  uint64_t empty[4];
  uint64_t accum;
  uint64_t never;  // nothing ever arrives here (time-out self-test)
  uint32_t tmem_base;
  int abort_flag;
  int row_perm[kMaxBN];       // permuted row of tile row j, or -1
  int prow[kMaxBN + 12];      // tile rows sorted by format, each format padded to four (-1)
  int nquad;                  // groups of four rows in prow
  float colscale[kMaxBN];
  float colbias[kMaxBN];
};

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::
          "r"(dst),
      "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
__device__ __forceinline__ uint64_t make_desc_sw128(uint32_t smem_addr) {
  // K-major, 128-byte swizzle: 8-row groups 1024 B apart; descriptor version 1
  uint64_t d = (smem_addr & 0x3ffffu) >> 4;
  d |= 1ull << 16;                                  // leading byte offset (unused for swizzled K-major)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;      // stride byte offset
  d |= 1ull << 46;                                  // version
  d |= 2ull << 61;                                  // SWIZZLE_128B
  return d;
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
      "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ uint4 ldg_nc16(const void *p) {
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t ldg_nc4(const void *p) {
  uint32_t v;
  asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}

// wait on a barrier unless the CTA is aborting; raises the abort flag on timeout
__device__ __forceinline__ bool gemm_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag) {
  for (int i = 0; i < 20000; ++i) {
    if (mbar_try(smem_u32(bar), parity, 50000u)) return true;
    if (*abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}

}  // namespace
}  // namespace rdq

#include "rdq_gemm_kernel.inl"
