// Kernel and launchers of rdq_gemv_tiled.cu (included at its end; see the header comment there).
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

__device__ __forceinline__ uint4 ldg_cg16(const void *p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
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
  int test_timeout;  // self-test: CTA 0 ends with a wait that runs out
  // Peer mode (column-parallel layers): the outputs go to n_dst destinations -- one slice of a
  // gather buffer on every GPU of the node, this one included, written with plain stores over
  // NVLink -- instead of y; the last epilogue warp of the grid then raises this rank's flag on
  // every GPU.  n_dst == 0: off.
  int n_dst;
  __half *dst[kMaxPeers];
  int32_t *peer_flag[kMaxPeers];  // this rank's flag word on every GPU
  int32_t *peer_state;            // local: [0] epilogue warps done in this launch, [1] launches completed
  // Activation prologue (0: x is used as it is).  1: x_in = x (+ x_aux); the CTA's activation rows
  // are f16(x_in * rsqrt(mean(x_in^2) + eps)) * x_weight, and CTA 0 writes x_in to x_out (the
  // updated residual stream).  2: x is [M, 2 K] and the rows are silu(x[:, :K]) * x[:, K:].
  int xop;
  const __half *x_aux;
  const __half *x_weight;
  __half *x_out;
  float x_eps;
};

constexpr int kStageUnroll = 2;  // pair-loop unrolling of the NVFP4 / FP8 stages

// Activation fragment loads: from the shared-memory copy (XS) or from global memory.
// `base` is a shared-memory byte address (XS) or a generic pointer value.
template <bool XS>
__device__ __forceinline__ uint4 ldx16(uint64_t base, int byte_off) {
  uint4 v;
  if (XS) {
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(static_cast<uint32_t>(base) + byte_off) : "memory");
  } else {
    v = t_ldx16(reinterpret_cast<const __half *>(base + byte_off));
  }
  return v;
}
template <bool XS>
__device__ __forceinline__ uint2 ldx8(uint64_t base, int byte_off) {
  uint2 v;
  if (XS) {
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];"
                 : "=r"(v.x), "=r"(v.y) : "r"(static_cast<uint32_t>(base) + byte_off) : "memory");
  } else {
    v = t_ldx8(reinterpret_cast<const __half *>(base + byte_off));
  }
  return v;
}
template <bool XS>
__device__ __forceinline__ uint32_t ldx4(uint64_t base, int byte_off) {
  uint32_t v;
  if (XS) {
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(static_cast<uint32_t>(base) + byte_off) : "memory");
  } else {
    v = t_ldx4(reinterpret_cast<const __half *>(base + byte_off));
  }
  return v;
}
__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
  return v;
}

// multiply-accumulate one NVFP4 piece (16 rows x 32 k): raw words of rows g / g+8, the
// E4M3 scale pair of the piece for each row (low 16 bits), the lane's 8 activations
template <int NT>
__device__ __forceinline__ void fp4_piece(float (&acc)[NT][2][4], uint32_t wg, uint32_t wg8, uint32_t sraw_g,
                                          uint32_t sraw_g8, uint32_t sel, const uint4 (&xv)[NT]) {
  const uint32_t sg = __byte_perm(cvt_e4m3x2(sraw_g), 0u, sel);
  const uint32_t sg8 = __byte_perm(cvt_e4m3x2(sraw_g8), 0u, sel);
  uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
  cvt_e2m1x8(wg, a0, a1, a2, a3);
  cvt_e2m1x8(wg8, b0, b1, b2, b3);
  a0 = hmul2_u32(a0, sg); a1 = hmul2_u32(a1, sg); a2 = hmul2_u32(a2, sg); a3 = hmul2_u32(a3, sg);
  b0 = hmul2_u32(b0, sg8); b1 = hmul2_u32(b1, sg8); b2 = hmul2_u32(b2, sg8); b3 = hmul2_u32(b3, sg8);
#pragma unroll
  for (int n = 0; n < NT; ++n) {
    mma_16816(acc[n][0], a0, b0, a1, b1, xv[n].x, xv[n].y);
    mma_16816(acc[n][1], a2, b2, a3, b3, xv[n].z, xv[n].w);
  }
}

// Per-lane shared-memory addresses inside a stage, for the pair of pieces the warp starts with.
// A "pair" is two 16-byte pieces of every row = one ldmatrix.x4.
//
// ---- NVFP4 stage: pairs [lo, hi) of 16 rows x 64 k.  All loads of a pair are issued
// before its first use; addresses advance by constants.
template <int NT, bool XS>
__device__ __forceinline__ void stage_fp4(float (&acc)[NT][2][4], uint32_t lm_addr, uint32_t sc_addr,
                                          uint32_t sc8_addr, const uint64_t (&xb)[NT], int xoff, int npairs,
                                          uint32_t sel) {
#pragma unroll kStageUnroll
  for (int i = 0; i < npairs; ++i) {
    uint32_t w[4];
    ldmatrix_x4(lm_addr, w[0], w[1], w[2], w[3]);
    const uint32_t s_g = lds_u32(sc_addr);    // scale bytes of pieces (p, p+1) for row g
    const uint32_t s_g8 = lds_u32(sc8_addr);  // ... for row g + 8
    uint4 x0[NT], x1[NT];
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      x0[n] = ldx16<XS>(xb[n], xoff);
      x1[n] = ldx16<XS>(xb[n], xoff + 64);
    }
    fp4_piece<NT>(acc, w[0], w[1], s_g, s_g8, sel, x0);
    fp4_piece<NT>(acc, w[2], w[3], s_g >> 16, s_g8 >> 16, sel, x1);
    lm_addr += 32;
    sc_addr += 4;
    sc8_addr += 4;
    xoff += 128;
  }
}

// ---- FP8 stage: pairs of 16 rows x 32 k
template <int NT, bool XS>
__device__ __forceinline__ void stage_fp8(float (&acc)[NT][2][4], uint32_t lm_addr, const uint64_t (&xb)[NT],
                                          int xoff, int npairs) {
#pragma unroll kStageUnroll
  for (int i = 0; i < npairs; ++i) {
    uint32_t w[4];
    ldmatrix_x4(lm_addr, w[0], w[1], w[2], w[3]);
    uint2 x0[NT], x1[NT];
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      x0[n] = ldx8<XS>(xb[n], xoff);
      x1[n] = ldx8<XS>(xb[n], xoff + 32);
    }
    uint32_t a0, a4, a2, a6, c0, c4, c2, c6;
    cvt_e4m3x4(w[0], a0, a4);
    cvt_e4m3x4(w[1], a2, a6);
    cvt_e4m3x4(w[2], c0, c4);
    cvt_e4m3x4(w[3], c2, c6);
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      mma_16816(acc[n][0], a0, a2, a4, a6, x0[n].x, x0[n].y);
      mma_16816(acc[n][1], c0, c2, c4, c6, x1[n].x, x1[n].y);
    }
    lm_addr += 32;
    xoff += 64;
  }
}

// ---- FP16 stage: pairs of 16 rows x 16 k (32 B per row = two 16-byte pieces = one MMA)
template <int NT, bool XS>
__device__ __forceinline__ void stage_fp16(float (&acc)[NT][2][4], uint32_t lm_addr, const uint64_t (&xb)[NT],
                                           int xoff, int npairs) {
  auto one = [&](int c) {
    uint32_t w[4];
    ldmatrix_x4(lm_addr, w[0], w[1], w[2], w[3]);
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      const uint32_t x0 = ldx4<XS>(xb[n], xoff);
      const uint32_t x1 = ldx4<XS>(xb[n], xoff + 16);
      mma_16816(acc[n][c], w[0], w[1], w[2], w[3], x0, x1);
    }
    lm_addr += 32;
    xoff += 32;
  };
  int i = 0;
#pragma unroll 1
  for (; i + 1 < npairs; i += 2) {
    one(0);
    one(1);
  }
  if (i < npairs) one(0);
}

// Stage list entry (one 32-bit word per image this CTA streams, in processing order):
//   bits 1:0 format, bit 2 "hand over after this stage", bits 10:3 chunk index inside the
//   tile, bits 12:11 the epilogue warp that finishes the tile, bits 31:13 image index relative
//   to the CTA's first image.
constexpr uint32_t kEntFlush = 4u;

// first image, image count and format of tile gtile
__device__ __forceinline__ void tile_geom(const TSched &sc, int gtile, int &first_img, int &S, int &fmt) {
  if (gtile < sc.t4) {
    fmt = 0; S = sc.S4; first_img = gtile * sc.S4;
  } else if (gtile < sc.t4 + sc.t8) {
    fmt = 1; S = sc.S8; first_img = sc.e4 + (gtile - sc.t4) * sc.S8;
  } else {
    fmt = 2; S = sc.S16; first_img = sc.e8 + (gtile - sc.t4 - sc.t8) * sc.S16;
  }
}

// NT = number of 8-row activation groups (1: M <= 8, 2: M <= 16)
// EXTRA: the launch has an activation prologue or peer destinations (compiled apart so that the
// plain launch carries none of that code)
template <int NT, bool XS, bool EXTRA>
__global__ void __launch_bounds__(kThreads, 2) gemv_tiled_kernel(const __grid_constant__ TiledArgs a,
                                                  const __grid_constant__ TSched sc) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ __align__(8) uint64_t bar_full[kMaxStages];
  __shared__ __align__(8) uint64_t bar_empty[kMaxStages];
  __shared__ __align__(8) uint64_t fl_full[kGroups][kEpiWarps][kFlushRing];
  __shared__ __align__(8) uint64_t fl_empty[kGroups][kEpiWarps][kFlushRing];
  __shared__ __align__(8) uint64_t bar_x;
  __shared__ __align__(8) uint64_t bar_never;  // nothing ever arrives here (time-out self-test)
  __shared__ float xred[EXTRA ? RDQ_MAX_GEMV_M : 1][kMmaWarps];  // activation prologue: per-warp sums of squares

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int K = a.K, M = a.M;
  const int N = a.n4 + a.n8 + a.n16;
  const int nst = a.nstages;
  // hand-over rings, one per (warp group, epilogue warp): kFlushRing slots of
  // [4 warps][16 rows][mp] partial sums; each ring has one writer group and one reader warp,
  // which both follow its barriers phase by phase
  const int mp = (M <= 3) ? M : ((M + 3) & ~3);  // M > 3: rows of four floats, read 16 B at a time
  const int vp = (M <= 4) ? 4 : 16;               // row pitch of an epilogue warp's staging tile
  const int nepi = a.nepi;      // epilogue warps in use (1..kEpiWarps)
  const int fdep = a.fdepth;    // slots per hand-over ring (1 or 2)
  const int gslot_floats = kWarpsPerGroup * kTileRows * mp;
  float *flush = reinterpret_cast<float *>(smem + nst * a.slot_bytes);
  int *meta_col = reinterpret_cast<int *>(flush + kGroups * nepi * fdep * gslot_floats);
  float *meta_scl = reinterpret_cast<float *>(meta_col + kMetaSegs * kTileRows);
  float *meta_bia = meta_scl + kMetaSegs * kTileRows;
  uint32_t *list = reinterpret_cast<uint32_t *>(meta_bia + kMetaSegs * kTileRows);
  uint32_t *segtab = list + kMaxList;
  float *vstage = reinterpret_cast<float *>(segtab + kMaxList);  // per epilogue warp: [16 rows][16] finished sums of a tile
  uint8_t *xsm = reinterpret_cast<uint8_t *>(vstage + kEpiWarps * kTileRows * vp);
  const int xpitch = 2 * a.K + 16;  // activation row pitch in shared memory: skewed against bank conflicts

  // lane L holds the first image of CTA bx + L (one call site for the 64-bit divisions)
  const int bnd = sc.boundary(static_cast<int>(blockIdx.x) + lane);
  const int s_begin = __shfl_sync(0xffffffffu, bnd, 0);
  const int s_end = __shfl_sync(0xffffffffu, bnd, 1);
  const int nimg = s_end - s_begin;
  const int first_tile = (nimg > 0) ? sc.tile_of_image(s_begin) : 0;
  const int nseg = (nimg > 0) ? (sc.tile_of_image(s_end - 1) - first_tile + 1) : 0;
  int32_t *status = a.flags + a.status_idx;
  const int ck = sc.ck;
  const int pitch = (ck >> 1) + 16;

  if (tid == 0) {
    for (int i = 0; i < nst; ++i) {
      mbar_init(smem_u32(&bar_full[i]), 1);
      mbar_init(smem_u32(&bar_empty[i]), kWarpsPerGroup);
    }
    for (int g = 0; g < kGroups; ++g)
      for (int j = 0; j < kEpiWarps; ++j)
        for (int i = 0; i < kFlushRing; ++i) {
          mbar_init(smem_u32(&fl_full[g][j][i]), kWarpsPerGroup);
          mbar_init(smem_u32(&fl_empty[g][j][i]), 1);
        }
    mbar_init(smem_u32(&bar_x), 1);
    mbar_init(smem_u32(&bar_never), 1);
    mbar_init_fence();
  }
  __syncthreads();
  // Let the next kernel in the stream become resident as early as possible; until this
  // grid completes it only fills its own shared-memory ring with weights.
  pdl_launch_dependents();
  if (nimg > kMaxList) {  // the launcher refuses such shapes; never reached
    if (tid == 0) atomicExch(status, 8);
    return;
  }

  const uint32_t smem_base = smem_u32(smem);

  if (warp == kMmaWarps) {
    // ==================================================================== producer
    // The whole warp first writes the stage list: the CTA's images in processing order --
    // the (possibly split) first tile, whose partial sums another CTA waits for, then the
    // (possibly split) last tile, which this CTA finishes, then the whole tiles in between.
    {
      int f0, S0, fmt0;
      tile_geom(sc, first_tile, f0, S0, fmt0);
      const int n0 = min(s_end, f0 + S0) - s_begin;  // images of the first tile
      int nl = 0;                                    // images of the last tile
      if (nseg >= 2) {
        int fl, Sl, fmtl;
        tile_geom(sc, first_tile + nseg - 1, fl, Sl, fmtl);
        nl = s_end - max(s_begin, fl);
      }
      auto rel_of = [&](int it) { return it < n0 ? it : (it < n0 + nl ? nimg - nl + (it - n0) : it - nl); };
      for (int it = lane; it < nimg; it += 32) {
        const int rel = rel_of(it);
        const int gt = sc.tile_of_image(s_begin + rel);
        int f, S, fmt;
        tile_geom(sc, gt, f, S, fmt);
        // position of the tile in processing order, and the epilogue warp that takes it
        const int idx = gt - first_tile;
        const int q = (idx == 0) ? 0 : (idx == nseg - 1 ? 1 : idx + 1);
        uint32_t e = static_cast<uint32_t>(fmt) | (static_cast<uint32_t>(s_begin + rel - f) << 3) |
                     (static_cast<uint32_t>(q % nepi) << 11) | (static_cast<uint32_t>(rel) << 13);
        // the group that takes this stage hands its sums over after its last stage of the tile;
        // its next stage sits three slots further, or in its first slot of the next round
        const int sl = it % nst;
        const int nxt = (sl + kGroups < nst) ? it + kGroups : it + (nst - sl) + sl % kGroups;
        if (nxt >= nimg || sc.tile_of_image(s_begin + rel_of(nxt)) != gt) e |= kEntFlush;
        list[it] = e;
      }
      __syncwarp();
    }
    if (lane != 0) return;
    // The ring is filled with weights first (they do not depend on the preceding kernel);
    // only then wait for that kernel and fetch the activations it produced.
    bool x_sent = false;
    auto send_x = [&]() {
      if (x_sent) return;
      x_sent = true;
      // Only this thread executes the grid-dependency wait; every other warp of the CTA
      // sleeps on bar_x, which completes after it (and after the activation copies).
      pdl_wait();
      const uint32_t bx = smem_u32(&bar_x);
      if (XS && (!EXTRA || a.xop == 0)) {
        mbar_arrive_expect_tx(bx, static_cast<uint32_t>(M) * 2u * K);
        for (int m = 0; m < M; ++m) bulk_g2s(smem_u32(xsm) + m * xpitch, a.x + 1ll * m * K, 2u * K, bx);
      } else {  // the MMA warps fetch (and transform) the activations themselves
        mbar_arrive(bx);
      }
    };
    int slot = 0, round = 0;
#pragma unroll 1
    for (int it = 0; it < nimg; ++it) {
      const uint32_t e = list[it];
      const uint32_t bytes = static_cast<uint32_t>((e & 3u) == 0 ? sc.img4 : sc.img8);
      if (round > 0) {
        send_x();
        if (!mbar_wait(smem_u32(&bar_empty[slot]), (round - 1) & 1)) {
          atomicExch(status, 1);
          return;
        }
      }
      const uint32_t full = smem_u32(&bar_full[slot]);
      mbar_arrive_expect_tx(full, bytes);
      bulk_g2s(smem_base + slot * a.slot_bytes, a.tiled + sc.image_offset(s_begin + static_cast<int>(e >> 13)), bytes,
               full);
      if (++slot == nst) { slot = 0; ++round; }
    }
    send_x();
    return;
  }

  if (warp > kMmaWarps) {
    // =============================================================== epilogue warps
    // The first nepi of them take the tile segments in turn: segment q (in processing
    // order) belongs to warp q % nepi.
    const int ej = warp - kMmaWarps - 1;
    if (ej >= nepi) return;
    float *vst = vstage + ej * kTileRows * vp;
    // output column, scale and bias of every row this CTA finishes: constants of the
    // layer, fetched up front so that finishing a tile needs no global round trip.  With
    // more than one epilogue warp the first builds the segment table and the others do this.
    if (ej > 0 || nepi == 1) {
      const int nmeta = min(nseg, kMetaSegs) * kTileRows;
      const int nload = (nepi == 1) ? 1 : nepi - 1;
      for (int base = (nepi == 1 ? 0 : ej - 1) * 128; base < nmeta; base += 128 * nload) {
        int col[4];
        float scl[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int item = base + u * 32 + lane;
          col[u] = 0;
          scl[u] = 1.f;
          if (item < nmeta) {
            const int gt = first_tile + (item >> 4);
            const int prow = gt * kTileRows + (item & 15);
            col[u] = a.perm ? a.perm[prow] : prow;
            scl[u] = (gt < sc.t4) ? a.global4 : (gt < sc.t4 + sc.t8 ? a.s8[prow - a.n4] : 1.f);
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int item = base + u * 32 + lane;
          if (item < nmeta) {
            meta_col[item] = col[u];
            meta_scl[item] = scl[u];
            meta_bia[item] = a.bias ? __half2float(a.bias[col[u]]) : 0.f;
          }
        }
      }
    }
    // Segment table: one word per tile segment, in processing order --
    //   bits 8:0 tile index inside the CTA, bit 9 "tile starts here", bit 10 "tile ends here",
    //   bits 13:11 warp groups that hold partial sums of it, bits 15:14 / 17:16 / 19:18 for
    //   each group the number (modulo 4) of hand-overs it made to this segment's epilogue
    //   warp before: ring slot = bit 0, barrier parity = bit 1.
    // Built by one whole warp: a prefix sum over lanes q, q - nepi, q - 2 nepi, ...
    if (ej == 0) {
      int f0, S0, fmt0;
      tile_geom(sc, first_tile, f0, S0, fmt0);
      const int n0 = min(s_end, f0 + S0) - s_begin;  // images of the first tile
      int nl = 0;                                    // images of the last tile
      if (nseg >= 2) {
        int fl, Sl, fmtl;
        tile_geom(sc, first_tile + nseg - 1, fl, Sl, fmtl);
        nl = s_end - max(s_begin, fl);
      }
      int carry[kEpiWarps];  // hand-over counts so far per epilogue warp: 10 bits per group
#pragma unroll
      for (int j = 0; j < kEpiWarps; ++j) carry[j] = 0;
      for (int base = 0; base < nseg; base += 32) {
        const int q = base + lane;
        const int qe = q % nepi;
        int inc = 0;
        uint32_t e = 0;
        if (q < nseg) {
          const int idx = tseg_order(q, nseg);
          int f, S, fmt;
          tile_geom(sc, first_tile + idx, f, S, fmt);
          const int ia = max(s_begin, f), ib = min(s_end, f + S);
          const int nstage = ib - ia;
          const int it0 = (q == 0) ? 0 : (q == 1 ? n0 : n0 + nl + (f - (s_begin + n0)));
          e = static_cast<uint32_t>(idx) | (ia == f ? 1u << 9 : 0u) | (ib == f + S ? 1u << 10 : 0u);
          // groups that take a stage of this tile: stage i sits in slot i % nst, group slot % 3
          int mask = 0;
          for (int i = 0; i < nstage && mask != (1 << kGroups) - 1; ++i) mask |= 1 << (((it0 + i) % nst) % kGroups);
#pragma unroll
          for (int g = 0; g < kGroups; ++g) {
            if ((mask >> g) & 1) {
              inc |= 1 << (10 * g);
              e |= 1u << (11 + g);
            }
          }
        }
        int x = inc;
        for (int off = nepi; off < 32; off <<= 1) {
          const int y = __shfl_up_sync(0xffffffffu, x, off);
          if (lane >= off) x += y;
        }
        int mycarry = carry[0];
#pragma unroll
        for (int j = 1; j < kEpiWarps; ++j)
          if (qe == j) mycarry = carry[j];
        const int before = x - inc + mycarry;
#pragma unroll
        for (int g = 0; g < kGroups; ++g) e |= static_cast<uint32_t>((before >> (10 * g)) & 3) << (14 + 2 * g);
        if (q < nseg) segtab[q] = e;
        // totals of this chunk per epilogue warp: held by the last lane of each residue class
#pragma unroll
        for (int j = 0; j < kEpiWarps; ++j) {
          if (j < nepi) {
            int last = 31 - (((base + 31) % nepi) - j + nepi) % nepi;
            carry[j] += __shfl_sync(0xffffffffu, x, last);
          }
        }
      }
    }
    // a split tile whose first image this CTA holds (only its last tile can be one): the
    // other parts come from the CTAs bx + 1 .. b_last, in that order
    int b_last = blockIdx.x;
    {
      int f, S, fmt;
      tile_geom(sc, first_tile + nseg - 1, f, S, fmt);
      const int s_last = f + S - 1;
      b_last += __popc(__ballot_sync(0xffffffffu, lane >= 1 && bnd <= s_last && bnd < sc.e16));
      if (lane == 0 && b_last >= static_cast<int>(blockIdx.x) + 31) atomicExch(status, 7);
    }
    // metadata and segment table are complete for all epilogue warps in use
    asm volatile("bar.sync 1, %0;" ::"r"(nepi * 32) : "memory");
    // y, workspace and flags belong to this launch only once the preceding grid is done
    if (!mbar_wait(smem_u32(&bar_x), 0)) {
      if (lane == 0) atomicExch(status, 6);
      return;
    }
    // work item = (row, quad of four activation rows): lane L takes item L, and item L + 32
    // when M > 8
    const int row = lane & 15;
    const int nitem = (M > 8) ? 2 : 1;
    float *ws_row = a.workspace + 1ll * blockIdx.x * 256 + row * 16;
#pragma unroll 1
    for (int q = ej; q < nseg; q += nepi) {
      const uint32_t e = segtab[q];
      const int idx = e & 511;
      const bool starts = (e >> 9) & 1, ends = (e >> 10) & 1;
#pragma unroll
      for (int g = 0; g < kGroups; ++g) {
        const int code = (e >> (14 + 2 * g)) & 3;  // hand-overs before, modulo 4
        const int fsl = (fdep == 2) ? (code & 1) : 0, fpar = (fdep == 2) ? (code >> 1) : (code & 1);
        if (((e >> (11 + g)) & 1) && !mbar_wait(smem_u32(&fl_full[g][ej][fsl]), fpar)) {
          if (lane == 0) atomicExch(status, 2);
          return;
        }
      }
      int col;
      float scl, bia;
      if (idx < kMetaSegs) {
        col = meta_col[idx * kTileRows + row];
        scl = meta_scl[idx * kTileRows + row];
        bia = meta_bia[idx * kTileRows + row];
      } else {
        const int gt = first_tile + idx;
        const int prow = gt * kTileRows + row;
        col = a.perm ? a.perm[prow] : prow;
        scl = (gt < sc.t4) ? a.global4 : (gt < sc.t4 + sc.t8 ? a.s8[prow - a.n4] : 1.f);
        bia = a.bias ? __half2float(a.bias[col]) : 0.f;
      }
      // Sum first and give the ring slots back at once: the barrier arrival is a release,
      // and behind a global store it would wait for that store to be acknowledged.
      if (M <= 3) {
        // up to three activation rows: scalar reads, lane = (row, m parity)
#pragma unroll 1
        for (int m = lane >> 4; m < M; m += 2) {
          float v = 0.f;
#pragma unroll
          for (int g = 0; g < kGroups; ++g) {
            if ((e >> (11 + g)) & 1) {
              const float *ring = flush + ((g * nepi + ej) * fdep + (fdep == 2 ? ((e >> (14 + 2 * g)) & 1) : 0)) * gslot_floats;
#pragma unroll
              for (int w = 0; w < kWarpsPerGroup; ++w) v += ring[(w * kTileRows + row) * mp + m];
            }
          }
          vst[row * vp + m] = v;
        }
      } else {
#pragma unroll 1
        for (int j = 0; j < nitem; ++j) {
          const int m0 = ((lane >> 4) + 2 * j) * 4;
          if (m0 < M) {
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int g = 0; g < kGroups; ++g) {
              if ((e >> (11 + g)) & 1) {
                const float *ring = flush + ((g * nepi + ej) * fdep + (fdep == 2 ? ((e >> (14 + 2 * g)) & 1) : 0)) * gslot_floats;
#pragma unroll
                for (int w = 0; w < kWarpsPerGroup; ++w) {
                  const float4 p = *reinterpret_cast<const float4 *>(ring + (w * kTileRows + row) * mp + m0);
                  v.x += p.x; v.y += p.y; v.z += p.z; v.w += p.w;
                }
              }
            }
            *reinterpret_cast<float4 *>(vst + row * vp + m0) = v;
          }
        }
      }
      __syncwarp();
      if (lane == 0) {
#pragma unroll
        for (int g = 0; g < kGroups; ++g)
          if ((e >> (11 + g)) & 1) mbar_arrive(smem_u32(&fl_empty[g][ej][fdep == 2 ? ((e >> (14 + 2 * g)) & 1) : 0]));
      }
      const int b_hi = (starts && !ends) ? b_last : static_cast<int>(blockIdx.x);
      bool ok = true;
#pragma unroll 1
      for (int m = lane >> 4; m < M; m += 2) {
        float v = vst[row * vp + m];
        if (!starts) {
          // continuation of a tile another CTA started: store the partial sums into this
          // CTA's workspace slot (idle words read 0xffffffff); the owner polls them
          // strong store: performed at L2 at once (a plain store may linger in this SM while
          // other warps of this CTA poll for another CTA's sums)
          asm volatile("st.relaxed.gpu.global.f32 [%0], %1;" ::"l"(ws_row + m), "f"(v) : "memory");
          continue;
        }
#pragma unroll 1
        for (int b = blockIdx.x + 1; b <= b_hi; ++b) {
          float *pw = a.workspace + 1ll * b * 256 + row * 16 + m;
          uint32_t bits = 0xffffffffu;
#pragma unroll 1
          for (int spin = 0; spin < 2000000 && bits == 0xffffffffu; ++spin) {
            asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(bits) : "l"(pw) : "memory");
            if (bits == 0xffffffffu) __nanosleep(200);
          }
          if (bits == 0xffffffffu) ok = false;
          v += __uint_as_float(bits);
          *pw = __uint_as_float(0xffffffffu);  // slot idle again
        }
        const __half h = __float2half_rn(fmaf(v, scl, bia));
        if (!EXTRA || a.n_dst == 0) {
          a.y[1ll * m * N + col] = h;
        } else {
          // the 16 rows of a tile are consecutive columns of the slice: the stores of the lanes
          // of one activation row fall into one 32-byte sector per destination
          for (int d = 0; d < a.n_dst; ++d) a.dst[d][1ll * m * N + col] = h;
        }
      }
      __syncwarp();  // vst is rewritten for the next tile
      if (__any_sync(0xffffffffu, !ok)) {
        if (lane == 0) atomicExch(status, 3);
        return;
      }
    }
    if (EXTRA && a.n_dst > 0) {
      // This warp's stores to the other GPUs are complete system-wide before it counts itself
      // done; the warp that completes the count publishes the launch number in this rank's flag
      // word on every GPU (release: fence, then the flag stores).
      __threadfence_system();
      __syncwarp();
      if (lane == 0) {
        const int expected = static_cast<int>(gridDim.x) * nepi;
        if (atomicAdd(a.peer_state, 1) == expected - 1) {
          __threadfence_system();
          const int launch = a.peer_state[1] + 1;
          a.peer_state[1] = launch;
          a.peer_state[0] = 0;
          for (int d = 0; d < a.n_dst; ++d)
            asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(a.peer_flag[d]), "r"(launch) : "memory");
        }
      }
    }
    if (a.test_timeout && blockIdx.x == 0 && ej == 0) {
      // Self-test of the time-out path: all work of this warp is done and nothing of this CTA
      // is in flight; wait (three suspended tries) on a barrier that nothing completes and
      // report the expired wait like any other.
      if (!mbar_wait(smem_u32(&bar_never), 0, 3u) && lane == 0) atomicExch(status, 9);
    }
    return;
  }

  // ==================================================================== MMA warps
  const int g = lane >> 2;  // fragment row / activation row
  const int t = lane & 3;   // fragment k group
  // ldmatrix.x4: lanes 0-7 / 8-15 address rows 0-7 / 8-15 of the first piece of a pair,
  // lanes 16-31 the same rows of the second piece
  const uint32_t lm_lane = ((lane & 7) + ((lane >> 3) & 1) * 8) * pitch + (lane >> 4) * 16;
  const int spitch = scale_pitch(ck);
  const uint32_t sc_lane = kTileRows * pitch + g * spitch;  // block scales of row g
  const uint32_t sel = (t & 2) ? 0x3232u : 0x1010u;          // this lane's 8 codes sit in block t >> 1
  const int npair = ck >> 6;                                 // pairs of 16-byte pieces per row
  const int grp = warp / kWarpsPerGroup, wq = warp % kWarpsPerGroup;

  float acc[NT][2][4];
#pragma unroll
  for (int n = 0; n < NT; ++n)
#pragma unroll
    for (int c = 0; c < 2; ++c)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[n][c][i] = 0.f;

  // x is produced by the preceding kernel: do not touch it before the producer thread has
  // seen that kernel complete (and, with XS, has copied the rows into shared memory).
  // The stage list is complete by then, too.
  if (!mbar_wait(smem_u32(&bar_x), 0)) {
    if (lane == 0) atomicExch(status, 6);
    return;
  }
  if (EXTRA && XS && a.xop != 0) {
    // ---- activation prologue: the twelve MMA warps build the CTA's activation rows in shared
    // memory from what the preceding kernels left in global memory (every CTA does the same work:
    // a few KB out of L2).  A row is cut into `cpr` chunks, one warp per chunk, and a lane has
    // four vectors (eight with x_aux) in flight: the cost is a few L2 round trips.
    const int nvec = K >> 3;  // 16-byte vectors per row
    const int cpr = M >= kMmaWarps ? 1 : kMmaWarps / M;
    const int per = (nvec + cpr - 1) / cpr;
    if (a.xop == 1) {
      for (int u = warp; u < M * cpr; u += kMmaWarps) {
        const int m = u / cpr, c = u - m * cpr;
        const int hi = min(nvec, (c + 1) * per);
        const __half *xr = a.x + 1ll * m * K;
        const __half *dr = a.x_aux ? a.x_aux + 1ll * m * K : nullptr;
        __half *orow = (a.x_out && blockIdx.x == 0) ? a.x_out + 1ll * m * K : nullptr;
        float ss = 0.f;
        for (int i0 = c * per + lane; i0 < hi; i0 += 128) {
          uint4 v[4], d[4];
#pragma unroll
          for (int q = 0; q < 4; ++q)
            if (i0 + 32 * q < hi) v[q] = ldg_cg16(xr + 8 * (i0 + 32 * q));
          if (dr) {
#pragma unroll
            for (int q = 0; q < 4; ++q)
              if (i0 + 32 * q < hi) d[q] = ldg_cg16(dr + 8 * (i0 + 32 * q));
          }
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int i = i0 + 32 * q;
            if (i >= hi) break;
            __half2 *hv = reinterpret_cast<__half2 *>(&v[q]);
            if (dr) {
              const __half2 *dh = reinterpret_cast<const __half2 *>(&d[q]);
#pragma unroll
              for (int j = 0; j < 4; ++j) hv[j] = __hadd2(hv[j], dh[j]);
            }
            if (orow) *reinterpret_cast<uint4 *>(orow + 8 * i) = v[q];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 f = __half22float2(hv[j]);
              ss += f.x * f.x + f.y * f.y;
            }
            *reinterpret_cast<uint4 *>(xsm + m * xpitch + 16 * i) = v[q];
          }
        }
        ss = warp_sum(ss);
        if (lane == 0) xred[m][c] = ss;
      }
      asm volatile("bar.sync 2, %0;" ::"r"(kMmaWarps * 32) : "memory");
      for (int u = warp; u < M * cpr; u += kMmaWarps) {
        const int m = u / cpr, c = u - m * cpr;
        const int hi = min(nvec, (c + 1) * per);
        float ss = 0.f;
        for (int w = 0; w < cpr; ++w) ss += xred[m][w];
        const float rs = rsqrtf(ss / K + a.x_eps);
        for (int i = c * per + lane; i < hi; i += 32) {
          uint4 v = *reinterpret_cast<uint4 *>(xsm + m * xpitch + 16 * i);
          const uint4 wv = *reinterpret_cast<const uint4 *>(a.x_weight + 8 * i);
          __half2 *hv = reinterpret_cast<__half2 *>(&v);
          const __half2 *wh = reinterpret_cast<const __half2 *>(&wv);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = __half22float2(hv[j]);
            hv[j] = __hmul2(__floats2half2_rn(f.x * rs, f.y * rs), wh[j]);
          }
          *reinterpret_cast<uint4 *>(xsm + m * xpitch + 16 * i) = v;
        }
      }
    } else {
      for (int u = warp; u < M * cpr; u += kMmaWarps) {
        const int m = u / cpr, c = u - m * cpr;
        const int hi = min(nvec, (c + 1) * per);
        const __half *gr = a.x + 2ll * m * K;
        for (int i0 = c * per + lane; i0 < hi; i0 += 128) {
          uint4 gv[4], uv[4];
#pragma unroll
          for (int q = 0; q < 4; ++q)
            if (i0 + 32 * q < hi) {
              gv[q] = ldg_cg16(gr + 8 * (i0 + 32 * q));
              uv[q] = ldg_cg16(gr + K + 8 * (i0 + 32 * q));
            }
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int i = i0 + 32 * q;
            if (i >= hi) break;
            const __half2 *gh = reinterpret_cast<const __half2 *>(&gv[q]);
            const __half2 *uh = reinterpret_cast<const __half2 *>(&uv[q]);
            uint4 o;
            __half2 *oh = reinterpret_cast<__half2 *>(&o);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 g2 = __half22float2(gh[j]);
              const __half2 sl = __floats2half2_rn(g2.x / (1.f + __expf(-g2.x)), g2.y / (1.f + __expf(-g2.y)));
              oh[j] = __hmul2(sl, uh[j]);
            }
            *reinterpret_cast<uint4 *>(xsm + m * xpitch + 16 * i) = o;
          }
        }
      }
    }
    asm volatile("bar.sync 2, %0;" ::"r"(kMmaWarps * 32) : "memory");
  }
  // Lanes of activation rows >= M read row 0 instead: their output columns are never stored.
  uint64_t xb[NT];
#pragma unroll
  for (int n = 0; n < NT; ++n) {
    const int m = n * 8 + g;
    xb[n] = XS ? static_cast<uint64_t>(smem_u32(xsm) + (m < M ? m : 0) * xpitch)
               : reinterpret_cast<uint64_t>(a.x + 1ll * (m < M ? m : 0) * K);
  }

  // Stage it sits in ring slot it % nst and goes to warp group slot % kGroups: a slot always
  // belongs to the same group, which therefore follows its barriers phase by phase whatever the
  // ring depth (a group that tested a barrier it had not followed could see a stale phase
  // parity, read the slot early and arrive twice on its empty barrier).
  float *fl_base = flush + grp * nepi * fdep * gslot_floats + wq * kTileRows * mp;
  int slot = grp, round = 0;
  int fcnt = 0;  // hand-overs made so far to each epilogue warp: 10 bits each
  int turn = 0;  // stages this group has taken: rotates the pair ranges among its warps
#pragma unroll 1
  for (int it = grp; it < nimg; ++turn) {
    const uint32_t e = list[it];
    if (!mbar_wait(smem_u32(&bar_full[slot]), round & 1)) {
      if (lane == 0) atomicExch(status, 4);
      return;
    }
    const uint32_t sbase = smem_base + slot * a.slot_bytes;
    const int c = (e >> 3) & 255;
    const int fmt = e & 3;
    // inside a group the warps take turns on the pair ranges, so uneven splits average out
    const int lw = (wq + turn) & (kWarpsPerGroup - 1);
    const int lo = lw * npair / kWarpsPerGroup, hi = (lw + 1) * npair / kWarpsPerGroup;
    if (fmt == 0) {
      stage_fp4<NT, XS>(acc, sbase + lm_lane + lo * 32, sbase + sc_lane + lo * 4, sbase + sc_lane + 8 * spitch + lo * 4,
                        xb, 2 * (c * ck + lo * 64 + t * 8), hi - lo, sel);
    } else if (fmt == 1) {
      stage_fp8<NT, XS>(acc, sbase + lm_lane + lo * 32, xb, 2 * (c * (ck >> 1) + lo * 32 + t * 4), hi - lo);
    } else {
      stage_fp16<NT, XS>(acc, sbase + lm_lane + lo * 32, xb, 2 * (c * (ck >> 2) + lo * 16 + t * 2), hi - lo);
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_u32(&bar_empty[slot]));
    if (slot + kGroups < nst) {
      slot += kGroups;
      it += kGroups;
    } else {  // on to the group's first slot, one round later
      it += nst - slot + grp;
      slot = grp;
      ++round;
    }

    if (e & kEntFlush) {
      // ---- the group's last stage of this tile: hand the partial sums to the tile's epilogue
      // warp, through the ring the two share
      const int ej = (e >> 11) & 3;
      const int cnt = (fcnt >> (10 * ej)) & 1023;
      fcnt += 1 << (10 * ej);
      const int fslot = (fdep == 2) ? (cnt & 1) : 0, fround = (fdep == 2) ? (cnt >> 1) : cnt;
      if (fround > 0 && !mbar_wait(smem_u32(&fl_empty[grp][ej][fslot]), (fround - 1) & 1)) {
        if (lane == 0) atomicExch(status, 5);
        return;
      }
      float *buf = fl_base + (ej * fdep + fslot) * gslot_floats;
#pragma unroll
      for (int n = 0; n < NT; ++n) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int r = g + (i >> 1) * 8;
          const int m = n * 8 + 2 * t + (i & 1);
          if (m < M) buf[r * mp + m] = acc[n][0][i] + acc[n][1][i];
          acc[n][0][i] = 0.f;
          acc[n][1][i] = 0.f;
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&fl_full[grp][ej][fslot]));
    }
  }
}

}  // namespace


void gemv_tiled_scratch(size_t *workspace_bytes, size_t *flag_bytes) {
  const int G = sm_count();
  *workspace_bytes = static_cast<size_t>(G) * 256 * sizeof(float);  // one partial tile per CTA
  *flag_bytes = (static_cast<size_t>(G) + 2) * sizeof(int32_t);     // status word at index G
}

// Shared-memory plan of one launch: weight ring | flush ring | output metadata | activations (if
// they fit).
struct SmemPlan {
  int nepi, fdep, nst, smem;
  bool xs;
};
static SmemPlan smem_plan(int M, int K) {
  SmemPlan p;
  const int slot_bytes = (img_bytes(0, tiled_chunk_k(K)) + 127) & ~127;
  // hand-over rings: (3 groups x nepi epilogue warps) x kFlushRing slots of 4 warps x 16 rows x
  // (M rounded up to 4) partial sums; fewer epilogue warps for large M keep this at 18-24 KB
  // up to four activation rows: 3 epilogue warps, 2-slot rings (18 KB at most); up to eight:
  // 3 warps, 1-slot rings (18 KB); beyond: 2 warps, 1-slot rings (24 KB)
  p.nepi = M <= 8 ? kEpiWarps : 2;
  p.fdep = M <= 4 ? kFlushRing : 1;
  const int mp = (M <= 3) ? M : ((M + 3) & ~3);
  const int fl_bytes = kGroups * p.nepi * p.fdep * kWarpsPerGroup * kTileRows * mp * 4;
  const int fixed = fl_bytes + kMetaSegs * kTileRows * 12 + kMaxList * 8 + kEpiWarps * kTileRows * (M <= 4 ? 4 : 16) * 4;
  const int total_budget = 112 * 1024;  // two CTAs (this layer's and the next one's) share an SM's 228 KB
  int xbytes = M * (2 * K + 16);
  p.xs = true;
  // Ring depth: slot s belongs to warp group s % 3, so depths 3k and 3k + 2 split the slots
  // 1:1:1 and (k+1):(k+1):k; 3k + 1 would leave one group with half as many more slots as the
  // others and measured slower than 3k.
  auto depth = [&](int xb) {
    int n = (total_budget - fixed - xb) / slot_bytes;
    if (n > kMaxStages) n = kMaxStages;
    return (n % kGroups == 1 && n > kGroups) ? n - 1 : n;
  };
  // activations go to shared memory while that leaves every warp group a ring slot: reading
  // them through L1 costs more than a shallower ring (measured for M = 3 .. 8)
  if (xbytes > 44 * 1024 || depth(xbytes) < min(kGroups, depth(0))) {
    p.xs = false;
    xbytes = 0;
  }
  p.nst = depth(xbytes);
  if (p.nst < kGroups) p.nst = kGroups;  // 3 x 19 KB always fits beside the fixed part
  p.smem = p.nst * slot_bytes + fixed + xbytes;
  return p;
}
bool tiled_stages_x(int M, int K) { return M >= 1 && M <= RDQ_MAX_GEMV_M && smem_plan(M, K).xs; }

int launch_gemv_tiled(const GemvTiledArgs &h, bool pdl, cudaStream_t stream) {
  const int ck = tiled_chunk_k(h.K);
  TSched sc;
  sc.ck = ck;
  sc.S4 = h.K / ck;
  sc.S8 = sc.S4 * 2;
  sc.S16 = sc.S4 * 4;
  sc.t4 = h.n4 / kTileRows;
  sc.t8 = h.n8 / kTileRows;
  const int t16 = h.n16 / kTileRows;
  sc.e4 = sc.t4 * sc.S4;
  sc.e8 = sc.e4 + sc.t8 * sc.S8;
  sc.e16 = sc.e8 + t16 * sc.S16;
  sc.img4 = img_bytes(0, ck);
  sc.img8 = img_bytes(1, ck);

  TiledArgs a;
  a.x = h.x; a.M = h.M; a.tiled = h.tiled; a.s8 = h.s8; a.global4 = h.global4; a.perm = h.perm;
  a.bias = h.bias; a.y = h.y; a.n4 = h.n4; a.n8 = h.n8; a.n16 = h.n16; a.K = h.K;
  a.workspace = h.workspace; a.flags = h.flags;
  a.test_timeout = h.test_timeout;
  a.n_dst = h.n_dst;
  for (int d = 0; d < kMaxPeers; ++d) {
    a.dst[d] = d < h.n_dst ? h.dst[d] : nullptr;
    a.peer_flag[d] = d < h.n_dst ? h.peer_flag[d] : nullptr;
  }
  a.peer_state = h.peer_state;
  a.xop = h.xop; a.x_aux = h.x_aux; a.x_weight = h.x_weight; a.x_out = h.x_out; a.x_eps = h.x_eps;
  a.status_idx = sm_count();
  a.slot_bytes = (img_bytes(0, ck) + 127) & ~127;
  const int nt = h.M <= 8 ? 1 : 2;
  const SmemPlan pl = smem_plan(h.M, h.K);
  a.nepi = pl.nepi;
  a.fdepth = pl.fdep;
  a.nstages = pl.nst;
  const bool xs = pl.xs;
  const int nst = pl.nst;
  RDQ_REQUIRE(h.xop == 0 || xs, RDQ_E_UNSUPPORTED,
              "activation prologue needs the activation rows in shared memory (M=%d, K=%d)", h.M, h.K);
  RDQ_REQUIRE(h.xop == 0 || (h.xop == 1 && h.x_weight) || h.xop == 2, RDQ_E_INVALID, "bad activation prologue");
  const int smem = pl.smem;

  // Images are balanced by what they cost a CTA in time, not by their bytes: an NVFP4 image
  // (conversion + block scaling) takes more instructions than an FP8 or FP16 image of the
  // same size, but images beyond the ring's depth mostly cost the wait for their copy.
  {
    // Time model of a CTA that streams n images of one format (cycles, three warp groups):
    // the first nst images are in the ring when the kernel may start and cost their compute
    // time c; each later one costs (landing time + c) / slots per group.  Find the common
    // finishing time T at which the three formats' images fill exactly the grid, and weigh
    // an image by 1 / n(T).
    // Constants measured on B200 with in-kernel clocks (compute) and fitted on the benchmark
    // block (landing time: 2500 .. 7000 give the same step time within 2 %, 1200 is 8 % slower).
    const double kappa[3] = {0.123, 0.0715, 0.038};  // compute cycles per image byte and group
    const double land = 4500.0;                      // cycles from copy issue to landing under load
    const double img[3] = {double(sc.img4), double(sc.img8), double(sc.img8)};
    const double cnt[3] = {double(sc.e4), double(sc.e8 - sc.e4), double(sc.e16 - sc.e8)};
    const double spg = double(nst) / kGroups;
    auto n_of = [&](int f, double T) {
      const double c = kappa[f] * img[f], p = (land + c) / spg;
      const double t_ring = nst * c / kGroups;
      return T <= t_ring ? T * kGroups / c : nst + (T - t_ring) * kGroups / p;
    };
    double lo = 1.0, hi = 1e9;
    for (int it = 0; it < 60; ++it) {
      const double T = 0.5 * (lo + hi);
      double ctas = 0;
      for (int f = 0; f < 3; ++f) ctas += cnt[f] / n_of(f, T);
      if (ctas > sm_count()) lo = T; else hi = T;
    }
    const double n4 = n_of(0, hi), n8 = n_of(1, hi), n16 = n_of(2, hi);
    sc.u4 = 1000;
    sc.u8 = max(1, min(1000, static_cast<int>(1000.0 * n4 / n8 + 0.5)));
    sc.u16 = max(1, min(sc.u8, static_cast<int>(1000.0 * n4 / n16 + 0.5)));
  }
  sc.w4 = 1ll * sc.e4 * sc.u4;
  sc.w8 = sc.w4 + 1ll * (sc.e8 - sc.e4) * sc.u8;
  sc.W = sc.w8 + 1ll * (sc.e16 - sc.e8) * sc.u16;
  // every CTA must own at least one image: its share may not be shorter than the
  // heaviest image
  int G = sm_count();
  // ... and a tile may spread over at most 31 CTAs (the owner finds them with one ballot)
  long long minshare = sc.u4;  // u4 is the largest cost
  const long long tile_cost[3] = {1ll * sc.S4 * sc.u4, 1ll * sc.S8 * sc.u8, 1ll * sc.S16 * sc.u16};
  for (int f = 0; f < 3; ++f)
    if ((tile_cost[f] + 29) / 30 > minshare) minshare = (tile_cost[f] + 29) / 30;
  const long long maxg = sc.W / minshare;
  if (maxg < G) G = static_cast<int>(maxg);
  if (G < 1) G = 1;
  sc.G = G;
  RDQ_REQUIRE(sc.W / G / sc.u16 + 2 <= kMaxList, RDQ_E_UNSUPPORTED,
              "layer too large for the tiled GEMV: more than %d images per CTA", kMaxList);

  static int smem_set[64][8] = {};
  static std::mutex smem_mutex;
  int dev = 0;
  RDQ_CUDA(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> smem_lock(smem_mutex);
  const bool extra = h.xop != 0 || h.n_dst > 0;
  const int variant = (extra ? 4 : 0) + (nt - 1) * 2 + (xs ? 1 : 0);
  static const void *const fns[8] = {
      reinterpret_cast<const void *>(gemv_tiled_kernel<1, false, false>),
      reinterpret_cast<const void *>(gemv_tiled_kernel<1, true, false>),
      reinterpret_cast<const void *>(gemv_tiled_kernel<2, false, false>),
      reinterpret_cast<const void *>(gemv_tiled_kernel<2, true, false>),
      reinterpret_cast<const void *>(gemv_tiled_kernel<1, false, true>),
      reinterpret_cast<const void *>(gemv_tiled_kernel<1, true, true>),
      reinterpret_cast<const void *>(gemv_tiled_kernel<2, false, true>),
      reinterpret_cast<const void *>(gemv_tiled_kernel<2, true, true>)};
  const void *fn = fns[variant];
  if (dev < 64 && smem_set[dev][variant] < smem) {
    RDQ_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    // Always the largest shared-memory carve-out: layers of different footprints follow each
    // other, and an SM cannot change its carve-out while a CTA of the previous layer is resident
    // (the next layer's CTA would wait instead of filling its ring alongside).
    RDQ_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
    smem_set[dev][variant] = smem;
  }

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(G));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  void *params[2] = {&a, &sc};
  RDQ_CUDA(cudaLaunchKernelExC(&cfg, fn, params));
  return RDQ_OK;
}


// ---------------------------------------------------------------------------------------
// Entry point for callers that cannot allocate device memory (no counterpart in the
// reference).  Its scratch -- the per-CTA partial-tile slots and the status word the
// tiled GEMV needs -- lives in the array below, which every GPU that loads this library
// holds until the process exits.  Sized for GPUs with up to kNoAllocMaxCtas SMs.
// ---------------------------------------------------------------------------------------
namespace {
constexpr int kNoAllocMaxCtas = 160;
constexpr int kNoAllocWsWords = kNoAllocMaxCtas * 256;  // workspace: one 16 x 16 float slot per CTA
constexpr int kNoAllocCntWords = kNoAllocMaxCtas + 32;                  // flags + status word
static __device__ __align__(256) uint32_t g_noalloc_scratch[kNoAllocWsWords + kNoAllocCntWords];

std::mutex g_noalloc_mutex;
void *g_noalloc_ptr[64] = {};

// Device address of the library array on the current device; the first call per device looks
// it up and puts the array into its idle state on `stream`.
int noalloc_array(void **out, cudaStream_t stream) {
  int dev = 0;
  RDQ_CUDA(cudaGetDevice(&dev));
  RDQ_REQUIRE(dev >= 0 && dev < 64, RDQ_E_UNSUPPORTED, "device index %d is beyond the 64 devices this entry point tracks", dev);
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (!g_noalloc_ptr[dev]) {
    // Set-up, once per device, with that device current.  In host code the array's name is
    // only a stand-in; the address a kernel can use has to come from the runtime.
    void *p = nullptr;
    RDQ_CUDA(cudaGetSymbolAddress(&p, g_noalloc_scratch));
    // idle partial-sum slots read 0xffffffff; flags and status word start at zero
    RDQ_CUDA(cudaMemsetAsync(p, 0xff, sizeof(uint32_t) * kNoAllocWsWords, stream));
    RDQ_CUDA(cudaMemsetAsync(static_cast<uint32_t *>(p) + kNoAllocWsWords, 0, sizeof(uint32_t) * kNoAllocCntWords, stream));
    g_noalloc_ptr[dev] = p;
  }
  *out = g_noalloc_ptr[dev];
  return RDQ_OK;
}

const char *tiled_status_text(int code) {
  switch (code) {
    case 1: return "producer: a ring slot was never released";
    case 2: return "epilogue: a warp group never handed over its partial sums";
    case 3: return "epilogue: another CTA never published its part of a split tile";
    case 4: return "MMA warps: a weight image never landed in the ring";
    case 5: return "MMA warps: a hand-over slot was never released";
    case 6: return "the activations were never staged (wait on the preceding kernel)";
    case 7: return "a tile is spread over more CTAs than the owner can collect";
    case 8: return "more images per CTA than the stage list holds";
    case 9: return "time-out self-test (RDQ_GEMV_TEST_TIMEOUT)";
    default: return "unknown status";
  }
}
}  // namespace

int gemv_tiled_noalloc(const GemvTiledArgs &in, bool pdl, cudaStream_t stream) {
  RDQ_REQUIRE(sm_count() <= kNoAllocMaxCtas, RDQ_E_UNSUPPORTED,
              "built-in scratch holds %d CTA slots but this GPU has %d SMs; use rdq_gemv_tiled with caller scratch",
              kNoAllocMaxCtas, sm_count());
  void *p = nullptr;
  const int rc = noalloc_array(&p, stream);
  if (rc != RDQ_OK) return rc;
  GemvTiledArgs a = in;
  a.workspace = static_cast<float *>(p);
  a.flags = reinterpret_cast<int32_t *>(static_cast<uint32_t *>(p) + kNoAllocWsWords);
  return launch_gemv_tiled(a, pdl, stream);
}

// Status word of the tiled GEMV after everything queued on `stream` has run: the caller's
// scratch pair, or (both null) the library array of the no-allocation entry point.  With
// `reset`, the status word and flags return to zero and every partial-sum slot to its idle
// pattern, so the next launch starts clean even after a launch that gave up a wait.
int gemv_tiled_status(float *workspace, int32_t *flags, bool reset, cudaStream_t stream) {
  size_t ws_bytes = 0, flag_bytes = 0;
  if (!workspace && !flags) {
    void *p = nullptr;
    const int rc = noalloc_array(&p, stream);
    if (rc != RDQ_OK) return rc;
    workspace = static_cast<float *>(p);
    flags = reinterpret_cast<int32_t *>(static_cast<uint32_t *>(p) + kNoAllocWsWords);
    ws_bytes = sizeof(uint32_t) * kNoAllocWsWords;
    flag_bytes = sizeof(uint32_t) * kNoAllocCntWords;
  } else {
    RDQ_REQUIRE(workspace && flags, RDQ_E_INVALID, "workspace and counters must both be given (or both null)");
    gemv_tiled_scratch(&ws_bytes, &flag_bytes);
  }
  int32_t code = 0;
  RDQ_CUDA(cudaMemcpyAsync(&code, flags + sm_count(), sizeof(code), cudaMemcpyDeviceToHost, stream));
  RDQ_CUDA(cudaStreamSynchronize(stream));
  if (reset) {
    RDQ_CUDA(cudaMemsetAsync(workspace, 0xff, ws_bytes, stream));
    RDQ_CUDA(cudaMemsetAsync(flags, 0, flag_bytes, stream));
  }
  RDQ_REQUIRE(code == 0, RDQ_E_DEVICE, "tiled GEMV: a bounded device-side wait ran out (status %d: %s); results of that launch are invalid",
              static_cast<int>(code), tiled_status_text(code));
  return RDQ_OK;
}

// ---------------------------------------------------------------------------------------
// Peer mode, receiving side: wait (bounded) until every rank's flag on this GPU shows the
// launch this call belongs to, then y[i] = buffer[index[i]] (un-permute out of the gather
// buffer).
// ---------------------------------------------------------------------------------------
namespace {
constexpr int kGatherThreads = 256;
__global__ void __launch_bounds__(kGatherThreads) peer_gather_kernel(const __half *buffer, const long long *index, __half *y,
                                                                    long long count, const int32_t *flags, int world,
                                                                    const int32_t *sent_state, int32_t *status, int wait_ms) {
  __shared__ int ok;
  // let the next layer's GEMV become resident now (it only fills its weight rings until this
  // kernel is complete), then wait for this layer's GEMV
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x == 0) ok = 1;
  __syncthreads();
  // the GEMV of this launch has completed on this GPU: its launch number is the one every
  // rank's flag must show
  const int launch = sent_state[1];
  if (threadIdx.x < world) {
    int v = 0;
    // about wait_ms milliseconds of 0.25 us naps
    for (long long spin = 0; spin < 4000ll * wait_ms; ++spin) {
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(flags + threadIdx.x) : "memory");
      if (v >= launch) break;
      __nanosleep(250);
    }
    if (v < launch) {
      ok = 0;
      atomicExch(status, 10 + static_cast<int>(threadIdx.x));  // 10 + rank that never arrived
    }
  }
  __syncthreads();
  if (!ok) return;
  const long long stride = 1ll * gridDim.x * blockDim.x;
  long long i = 1ll * blockIdx.x * blockDim.x + threadIdx.x;
  for (; i + 3 * stride < count; i += 4 * stride) {  // four independent index -> value chains in flight
    const long long j0 = index[i], j1 = index[i + stride], j2 = index[i + 2 * stride], j3 = index[i + 3 * stride];
    const __half v0 = buffer[j0], v1 = buffer[j1], v2 = buffer[j2], v3 = buffer[j3];
    y[i] = v0; y[i + stride] = v1; y[i + 2 * stride] = v2; y[i + 3 * stride] = v3;
  }
  for (; i < count; i += stride) y[i] = buffer[index[i]];
}
}  // namespace

int launch_peer_gather(const __half *buffer, const long long *index, __half *y, long long count, const int32_t *flags,
                       int world, const int32_t *sent_state, int32_t *status, int wait_ms, bool pdl, cudaStream_t stream) {
  // one CTA per SM, each with the footprint that keeps a second one off its SM (pin_slot); every
  // CTA waits for the flags, so none leaves before the GEMV after this kernel has its CTAs placed
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(sm_count()));
  cfg.blockDim = dim3(kGatherThreads);
  cfg.dynamicSmemBytes = kSlotSmem;
  cfg.stream = stream;
  RDQ_CUDA(pin_slot(reinterpret_cast<const void *>(peer_gather_kernel), kSlotSmem));
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  RDQ_CUDA(cudaLaunchKernelEx(&cfg, peer_gather_kernel, buffer, index, y, count, flags, world, sent_state, status, wait_ms));
  return RDQ_OK;
}

}  // namespace rdq
