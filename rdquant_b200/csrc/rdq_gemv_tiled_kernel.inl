// Kernel part of rdq_gemv_tiled.cu (included at its end; see the header comment there).
namespace rdq {

namespace {

// Image schedule, identical on every CTA.  Images are numbered in storage order.
struct TSched {
  int ck;            // chunk length in NVFP4 elements
  int S4, S8, S16;   // images per tile in each group
  int t4, t8;        // tiles in the NVFP4 / FP8 groups
  int e4, e8, e16;   // end of each group's image range
  int u4, u8, u16;   // scheduling cost of one NVFP4 / FP8 / FP16 image
  int img4, img8;    // image bytes (FP8 and FP16 images have the same size)
  long long w4, w8, W;
  int G;

  __device__ __forceinline__ int image_of_pos(long long p) const {
    if (p < w4) return static_cast<int>(p / u4);
    if (p < w8) return e4 + static_cast<int>((p - w4) / u8);
    if (p < W) return e8 + static_cast<int>((p - w8) / u16);
    return e16;
  }
  __device__ __forceinline__ int boundary(int b) const {
    if (b >= G) return e16;
    return image_of_pos(W * b / G);
  }
  __device__ __forceinline__ int tile_of_image(int s) const {
    if (s < e4) return s / S4;
    if (s < e8) return t4 + (s - e4) / S8;
    return t4 + t8 + (s - e8) / S16;
  }
  // byte offset of image s inside the tiled buffer
  __device__ __forceinline__ long long image_offset(int s) const {
    if (s < e4) return 1ll * s * img4;
    return 1ll * e4 * img4 + 1ll * (s - e4) * img8;
  }
};

// processing order of a CTA's tile segments: the (possibly split) first tile, whose
// partial another CTA is waiting for, then the (possibly split) last tile, which this
// CTA finishes, then the whole tiles in between
__device__ __forceinline__ int tseg_order(int q, int nseg) {
  if (q == 0) return 0;
  if (q == 1) return nseg - 1;
  return q - 1;
}

// x is written by the preceding kernel: coherent loads, issued only after the PDL wait
__device__ __forceinline__ uint4 t_ldx16(const __half *p) {
  uint4 v;
  asm volatile("ld.global.L1::evict_last.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint2 t_ldx8(const __half *p) {
  uint2 v;
  asm volatile("ld.global.L1::evict_last.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t t_ldx4(const __half *p) {
  uint32_t v;
  asm volatile("ld.global.L1::evict_last.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

struct TiledArgs {
  const __half *x;
  int M;
  const uint8_t *tiled;
  const float *s8;
  float global4;
  const int32_t *perm;
  const __half *bias;
  __half *y;
  int n4, n8, n16, K;
  float *workspace;
  int32_t *flags;  // one per CTA, then the status word at index status_idx
  int status_idx;
  int nstages;
  int slot_bytes;
  int nepi;    // epilogue warps in use
  int fdepth;  // slots per hand-over ring
};

#ifdef RDQ_TIMELINE
__device__ long long g_ttimeline[4 * 148 * 32];
__device__ int g_tl_base_dummy;
#define g_tl_base (((ttl_m - 1) & 3) * 148 * 32)
__device__ __forceinline__ void ttl_mark_(int slot, int ttl_m) {
  long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  if (blockIdx.x < 148 && slot < 32) g_ttimeline[g_tl_base + blockIdx.x * 32 + slot] = t;
}
// launches of the benchmark block are told apart by their shapes (debug build only)
#define TTL_ID (a.K == 2560 ? (a.n4 + a.n8 + a.n16 > 10000 ? 3 : 1) : (a.K == 4096 ? 2 : 4))
#define TTL_MARK(slot) do { if ((threadIdx.x & 31) == 0) ttl_mark_(slot, TTL_ID); } while (0)
// fine-grained per-stage clocks of two CTAs of the M == 3 launch
__device__ long long g_tstage[2 * 48 * 8];
#define TST(idx_, col_) do { if (a.n4 + a.n8 + a.n16 > 15000 && (blockIdx.x == 10 || blockIdx.x == 100) && (idx_) < 48) \
  g_tstage[((blockIdx.x == 100) * 48 + (idx_)) * 8 + (col_)] = clock64(); } while (0)
#else
#define TST(idx_, col_) do { } while (0)
#define TTL_MARK(slot) do { } while (0)
#endif

}  // namespace
}  // namespace rdq

#include "rdq_gemv_tiled_kernel2.inl"
