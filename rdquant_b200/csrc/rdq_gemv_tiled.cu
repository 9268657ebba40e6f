// Decode GEMV (M <= 16) on the TILED weight layout: the sm_100a fast path.
//
// Layout (built once per layer by rdq_gemv_repack from the row-major checkpoint
// tensors).  Rows are grouped in tiles of 16 permuted rows, k in chunks of `ck`
// NVFP4 elements (ck/2 FP8, ck/4 FP16 elements: the same P = ck/2 bytes per row).
// Each (tile, chunk) is stored as one contiguous IMAGE of exactly the bytes a
// shared-memory stage holds:
//     16 rows x (P payload + 16 B skew)           [+ NVFP4: 16 skewed rows of ck/16 block scales]
// images of a tile are consecutive, tiles are consecutive, groups follow each
// other NVFP4 | FP8 | FP16.  The 16-byte skew makes the row pitch an odd multiple
// of 16 B, so ldmatrix reads of 8 rows never collide on a bank.
//
// Kernel: images are numbered in storage order and each CTA takes a contiguous,
// time-balanced range of them (a small model of ring-resident and streamed images per format,
// see launch_gemv_tiled).  Inside a CTA
//   producer warp   writes the CTA's stage list (one word per image: format, chunk, "hand
//                   over after this stage"), then one thread issues one cp.async.bulk
//                   (TMA) copy per image (10-19 KB) into a shared-memory ring, mbarrier
//                   tracked.  It starts BEFORE griddepcontrol.wait: under programmatic
//                   dependent launch the ring of this layer fills while the preceding
//                   kernel runs.  It is also the only thread that executes that wait; the
//                   other warps sleep on an mbarrier it completes once the activations are
//                   staged.
//   12 MMA warps    in 3 groups of 4; stage i goes to group i % 3, whose warps split its k
//                   pieces: ldmatrix the packed bytes, convert with the hardware
//                   E2M1 / E4M3 -> f16 converters, scale NVFP4 by its block scale (exact
//                   in f16) and issue mma.sync m16n8k16 with the 16 weight rows as the row
//                   operand and the activation rows as the 8-column operand; FP32
//                   accumulators.  A group's loop per stage is: read the list word, wait,
//                   compute, release the slot; after its last stage of a tile it writes its
//                   four partial sums into its own small ring.  Measured on B200 the
//                   NVFP4 stages run within 20 % of the E2M1 converter's throughput
//                   (one warp instruction per 4 cycles and scheduler).
//   epilogue warp   builds a segment table (which groups hold sums of which tile, and in
//                   which ring slot) with a warp prefix sum, then per tile adds the
//                   groups' partial sums in a fixed order, gives the slots back, applies
//                   FP8 channel scale + bias and stores y[m, perm[row]].
// A tile whose images are split between CTAs is finished by the CTA holding its
// first image.  The others store their partial sums into per-CTA workspace slots
// whose idle content is the word 0xffffffff; the owner polls the words it needs
// until they differ from that (bounded), sums them in CTA order (bitwise
// reproducible) and writes 0xffffffff back, so the workspace is idle again when
// the launch ends.  No fence or flag round trip sits on the publishing side.
//
// Algorithmic traffic per launch: n4*(K/2 + K/16) + n8*(K + 4) + n16*2K bytes
// (the skew adds 16 B per P payload bytes on top, 1.2-2.5 %).
//
// Reference behaviour replaced: the Marlin-repacked split-K family K2-K7 of
// rdquant/csrc/fused_gemv.cu (:1244-1969; repack rdquant/fused_gemv_pack.py:151-172).
#include "rdq_kernels.cuh"

namespace rdq {

namespace {

constexpr int kTileRows = 16;
constexpr int kMmaWarps = 12;
constexpr int kGroups = 3;          // warp groups; stage i is consumed by group i % 3
constexpr int kWarpsPerGroup = 4;   // power of two
static_assert(kGroups * kWarpsPerGroup == kMmaWarps, "warp groups must cover the MMA warps");
constexpr int kEpiWarps = 3;
constexpr int kThreads = (kMmaWarps + 1 + kEpiWarps) * 32;  // + producer warp + epilogue warps = 4 warpgroups
// 512 threads: the launch bounds ask for two CTAs (this layer's and the next one's) per SM,
// i.e. 64 registers per thread
constexpr int kFlushRing = 2;  // slots of a hand-over ring (one per warp group and epilogue warp)
constexpr int kMetaSegs = 16;       // tiles per CTA whose output metadata is preloaded into shared memory
constexpr int kMaxStages = 12;
constexpr int kChunkMax = 2048;  // longest k chunk of an image, in NVFP4 elements
constexpr int kMaxList = 256;       // images one CTA can stream (stage list entries)

// pitch of a block-scale row inside an NVFP4 image: the payload (ck / 16 bytes) rounded up to
// an odd multiple of 16 B, so that the eight rows a warp reads together fall on distinct banks
__host__ __device__ inline int scale_pitch(int ck) {
  int sp = ((ck >> 4) + 15) & ~15;
  if (((sp >> 4) & 1) == 0) sp += 16;
  return sp;
}
__host__ __device__ inline int img_bytes(int fmt, int ck) {
  const int pitch = (ck >> 1) + 16;
  return kTileRows * pitch + (fmt == 0 ? kTileRows * scale_pitch(ck) : 0);
}

}  // namespace

// Chunk length (in NVFP4 elements) for a given K, or 0 when K cannot be tiled:
// the smallest number of chunks n with K/n <= 2048 and K/n a multiple of 64.
int tiled_chunk_k(int K) {
  if (K <= 0 || K % 64 != 0) return 0;
  for (int n = (K + kChunkMax - 1) / kChunkMax; n <= K / 64; ++n) {
    if (K % n == 0 && (K / n) % 64 == 0) return K / n;
  }
  return 0;
}

bool tiled_supported(int n4, int n8, int n16, int K) {
  const int ck = tiled_chunk_k(K);
  if (ck == 0) return false;
  if ((n4 % kTileRows) || (n8 % kTileRows) || (n16 % kTileRows)) return false;
  // a stage-list entry holds the chunk index of an image inside its tile in 8 bits: awkward K
  // (short chunks) with more images per tile than that run on the any-shape kernel
  const int s4 = K / ck;
  if ((n16 > 0 && 4 * s4 > 256) || (n8 > 0 && 2 * s4 > 256) || (n4 > 0 && s4 > 256)) return false;
  return n4 + n8 + n16 > 0;
}

size_t tiled_bytes(int n4, int n8, int n16, int K) {
  const int ck = tiled_chunk_k(K);
  if (ck == 0) return 0;
  const size_t s4 = K / ck;
  return static_cast<size_t>(n4 / kTileRows) * s4 * img_bytes(0, ck) +
         static_cast<size_t>(n8 / kTileRows) * s4 * 2 * img_bytes(1, ck) +
         static_cast<size_t>(n16 / kTileRows) * s4 * 4 * img_bytes(2, ck);
}

namespace {

// ---------------------------------------------------------------------------
// repack: row-major checkpoint tensors -> tiled images (one thread per 16 bytes)
// ---------------------------------------------------------------------------
struct RepackArgs {
  const uint8_t *w4, *s4, *w8, *w16;
  uint8_t *out;
  int n4, n8, n16, K, ck;
};

__global__ void __launch_bounds__(256) repack_kernel(RepackArgs a) {
  const int ck = a.ck, P = ck >> 1, pitch = P + 16, SP = ck >> 4, spitch = scale_pitch(ck);
  const int S4 = a.K / ck;
  const long long img4 = img_bytes(0, ck), img8 = img_bytes(1, ck);
  const long long tot4 = 1ll * (a.n4 / kTileRows) * S4 * img4;
  const long long tot8 = 1ll * (a.n8 / kTileRows) * S4 * 2 * img8;
  const long long tot16 = 1ll * (a.n16 / kTileRows) * S4 * 4 * img8;
  const long long units = (tot4 + tot8 + tot16) >> 4;
  for (long long u = 1ll * blockIdx.x * blockDim.x + threadIdx.x; u < units;
       u += 1ll * gridDim.x * blockDim.x) {
    long long off = u << 4;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (off < tot4) {
      const long long img = off / img4;
      const int in = static_cast<int>(off - img * img4);
      const int tile = static_cast<int>(img / S4), c = static_cast<int>(img - 1ll * tile * S4);
      if (in < kTileRows * pitch) {
        const int r = in / pitch, b = in - r * pitch;
        if (b < P)
          v = *reinterpret_cast<const uint4 *>(a.w4 + (1ll * tile * kTileRows + r) * (a.K >> 1) + 1ll * c * P + b);
      } else {
        const int in2 = in - kTileRows * pitch;
        const int r = in2 / spitch, b = in2 - r * spitch;
        if (b < SP) {
          // SP is a multiple of 4 (ck % 64 == 0) but not always of 16: copy by words
          const uint8_t *src = a.s4 + (1ll * tile * kTileRows + r) * (a.K >> 4) + 1ll * c * SP + b;
          uint32_t w[4] = {0u, 0u, 0u, 0u};
          for (int i = 0; i < 4; ++i)
            if (b + 4 * i < SP) w[i] = *reinterpret_cast<const uint32_t *>(src + 4 * i);
          v = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
    } else {
      const bool is8 = off < tot4 + tot8;
      const long long o2 = off - tot4 - (is8 ? 0 : tot8);
      const int S = is8 ? S4 * 2 : S4 * 4;
      const long long img = o2 / img8;
      const int in = static_cast<int>(o2 - img * img8);
      const int tile = static_cast<int>(img / S), c = static_cast<int>(img - 1ll * tile * S);
      const int r = in / pitch, b = in - r * pitch;
      if (b < P) {
        const long long row = 1ll * tile * kTileRows + r;
        const uint8_t *src = is8 ? a.w8 + row * a.K + 1ll * c * P + b
                                 : a.w16 + row * a.K * 2 + 1ll * c * P + b;
        v = *reinterpret_cast<const uint4 *>(src);
      }
    }
    *reinterpret_cast<uint4 *>(a.out + off) = v;
  }
}

}  // namespace

int launch_repack(const void *w_fp4, const void *w_fp4_scales, const void *w_fp8, const void *w_fp16,
                  void *tiled_out, int n4, int n8, int n16, int K, cudaStream_t stream) {
  RepackArgs a;
  a.w4 = static_cast<const uint8_t *>(w_fp4);
  a.s4 = static_cast<const uint8_t *>(w_fp4_scales);
  a.w8 = static_cast<const uint8_t *>(w_fp8);
  a.w16 = static_cast<const uint8_t *>(w_fp16);
  a.out = static_cast<uint8_t *>(tiled_out);
  a.n4 = n4; a.n8 = n8; a.n16 = n16; a.K = K;
  a.ck = tiled_chunk_k(K);
  const size_t units = tiled_bytes(n4, n8, n16, K) / 16;
  if (units == 0) return RDQ_OK;
  size_t blocks = (units + 255) / 256;
  const size_t cap = static_cast<size_t>(sm_count()) * 16;
  if (blocks > cap) blocks = cap;
  repack_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(a);
  RDQ_CUDA(cudaGetLastError());
  return RDQ_OK;
}

}  // namespace rdq

#include "rdq_gemv_tiled_kernel.inl"
