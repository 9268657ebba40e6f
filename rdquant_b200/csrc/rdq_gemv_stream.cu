// Decode GEMV (M <= 16), stream kernel for sm_100a.
//
// One launch streams the NVFP4, FP8 and FP16 row groups of a layer exactly once
// from HBM.  The work is cut into "slices" of 16 permuted rows x 256 k; slices
// are numbered tile-major (all k of a 16-row tile, then the next tile; NVFP4
// tiles, then FP8, then FP16) and each CTA takes one contiguous, byte-balanced
// range of them (slice weights 9 : 16 : 32 = bytes of a 16x256 slice incl.
// block scales, in units of 256 B).  Inside a CTA:
//
//   L2 prefetch     before griddepcontrol.wait the CTA asks the TMA unit to pull
//                   its whole byte range into L2 (cp.async.bulk.prefetch.L2), so
//                   under programmatic dependent launch the weights of this
//                   layer stream from HBM while the preceding kernel still runs.
//   8 MMA warps     the k range of each 16-row tile segment is cut into batches
//                   (16 rows x 512/256/128 k = 4 KB of weights); batches go round
//                   robin to the warps.  A lane loads 64 contiguous bytes of row
//                   g and of row g+8 straight into registers in the order the
//                   tensor-core fragment wants (the k order inside a batch is
//                   permuted identically for x), converts with the hardware
//                   E2M1 / E4M3 -> f16 converters, scales NVFP4 by its block
//                   scale (exact in f16) and issues mma.sync m16n8k16: weights
//                   are the 16-row operand, the activation rows the 8-column
//                   operand, accumulation in FP32.
//   epilogue warp   per tile segment the 8 partial accumulators are summed in a
//                   fixed order through a 4-deep shared-memory ring; FP8 channel
//                   scale and bias are applied and y[m, perm[row]] is stored.
//
// A tile whose slices are split between CTAs is finished by the CTA that holds
// its first slice: the other CTAs publish their partial sums to the scratch
// workspace and raise a flag, the owner waits for the flags (bounded), sums the
// partials in CTA order (bitwise reproducible) and lowers the flags again.  A
// CTA works on its split tiles first so that this hand-over overlaps the rest
// of its stream.  Every wait is bounded; a wait that runs out sets the status
// word.
//
// Algorithmic traffic per launch: n4*(K/2 + K/16) + n8*(K + 4) + n16*2K bytes.
//
// Reference behaviour replaced: kernels K1-K7 of rdquant/csrc/fused_gemv.cu
// (:1198-1969) and the FP16-group F.linear + cat + index_select of
// rdquant/ops.py:60-63.
#include "rdq_kernels.cuh"

namespace rdq {

namespace {

constexpr int kTileRows = 16;
constexpr int kSliceK = 256;
constexpr int kMmaWarps = 8;
constexpr int kThreads = (kMmaWarps + 1) * 32;
constexpr int kMetaSegs = 32;                          // segments whose output metadata is staged in smem
constexpr int kUnit4 = 9, kUnit8 = 16, kUnit16 = 32;

// Static description of the slice schedule; identical on every CTA.
struct Sched {
  int S;            // slices per tile (K / 256)
  int t4, t8;       // tiles in the NVFP4 / FP8 groups
  int e4, e8, e16;  // end of the NVFP4 / FP8 / FP16 slice ranges (global slice numbering)
  long long w4, w8, W;  // cumulative weights
  int G;

  __device__ __forceinline__ int slice_of_pos(long long p) const {
    if (p < w4) return static_cast<int>(p / kUnit4);
    if (p < w8) return e4 + static_cast<int>((p - w4) / kUnit8);
    if (p < W) return e8 + static_cast<int>((p - w8) / kUnit16);
    return e16;
  }
  __device__ __forceinline__ long long pos_of_slice(int s) const {
    if (s < e4) return 1ll * s * kUnit4;
    if (s < e8) return w4 + 1ll * (s - e4) * kUnit8;
    return w8 + 1ll * (s - e8) * kUnit16;
  }
  // first slice of CTA b (b == G gives the end)
  __device__ __forceinline__ int boundary(int b) const {
    if (b >= G) return e16;
    return slice_of_pos(W * b / G);
  }
  __device__ int cta_of_slice(int s) const {
    int b = static_cast<int>(pos_of_slice(s) * G / W);
    if (b >= G) b = G - 1;
    while (b + 1 < G && boundary(b + 1) <= s) ++b;
    while (b > 0 && boundary(b) > s) --b;
    return b;
  }
};

// The part of one 16-row tile that this CTA streams.
struct Seg {
  int fmt;     // 0 NVFP4, 1 FP8, 2 FP16
  int gtile;   // tile index over all groups
  int row0;    // first row inside the format group
  int k0, k1;  // element range along k
  int nb;      // batches (512 / 256 / 128 k each)
  bool starts, ends;  // covers the first / last slice of its tile
  bool complete;
};

__device__ __forceinline__ Seg seg_at(const Sched &sc, int s_begin, int s_end, int gtile) {
  Seg sg;
  const int ts = gtile * sc.S;
  const int a = max(s_begin, ts), b = min(s_end, ts + sc.S);
  sg.gtile = gtile;
  sg.k0 = (a - ts) * kSliceK;
  sg.k1 = (b - ts) * kSliceK;
  sg.starts = (a == ts);
  sg.ends = (b == ts + sc.S);
  sg.complete = sg.starts && sg.ends;
  if (ts < sc.e4) {
    sg.fmt = 0; sg.row0 = gtile * kTileRows;
  } else if (ts < sc.e8) {
    sg.fmt = 1; sg.row0 = (gtile - sc.t4) * kTileRows;
  } else {
    sg.fmt = 2; sg.row0 = (gtile - sc.t4 - sc.t8) * kTileRows;
  }
  const int bk = 512 >> sg.fmt;
  sg.nb = (sg.k1 - sg.k0 + bk - 1) / bk;
  return sg;
}
// processing order of a CTA's segments: the (possibly split) first tile, whose partial
// another CTA is waiting for, then the (possibly split) last tile, which this CTA
// finishes, then the whole tiles in between
__device__ __forceinline__ int seg_order(int q, int nseg) {
  if (q == 0) return 0;
  if (q == 1) return nseg - 1;
  return q - 1;
}
__device__ __forceinline__ void st_release_gpu(int32_t *p, int32_t v) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int32_t ld_acquire_gpu(const int32_t *p) {
  int32_t v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ uint4 ldg_stream(const void *p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::evict_first.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint2 ldg_stream8(const void *p) {
  uint2 v;
  asm volatile("ld.global.nc.L1::evict_first.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}
// x is written by the preceding kernel: plain (coherent) loads, issued after the PDL wait
__device__ __forceinline__ uint4 ld_x16(const __half *p) {
  uint4 v;
  asm volatile("ld.global.L1::evict_last.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ float ld_cg_f32(const float *p) {
  float v;
  asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void l2_prefetch(const void *p, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

#ifdef RDQ_TIMELINE
__device__ long long g_timeline[148 * 32];
__device__ __forceinline__ void tl_mark(int slot) {
  long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  if (blockIdx.x < 148 && slot < 32) g_timeline[blockIdx.x * 32 + slot] = t;
}
#define TL_MARK(slot) do { if ((threadIdx.x & 31) == 0) tl_mark(slot); } while (0)
#else
#define TL_MARK(slot) do { } while (0)
#endif

template <int NT>
struct XRows {
  const __half *row[NT];
  bool valid[NT];
};

// ---- one batch of NVFP4: 16 rows x 512 k; this lane owns k_t .. k_t+127 of rows g, g+8
template <int NT>
__device__ __forceinline__ void batch_fp4(float (&acc)[NT][2][4], const GemvArgs &a, const XRows<NT> &xr,
                                          int row, int k_t, bool tv) {
  const int K = a.K;
  uint4 wg[4], wh[4];
  uint2 sg = make_uint2(0u, 0u), sh = make_uint2(0u, 0u);
  if (tv) {
    const uint8_t *pg = a.w4 + 1ll * row * (K >> 1) + (k_t >> 1);
    const uint8_t *ph = pg + 8ll * (K >> 1);
#pragma unroll
    for (int i = 0; i < 4; ++i) wg[i] = ldg_stream(pg + 16 * i);
#pragma unroll
    for (int i = 0; i < 4; ++i) wh[i] = ldg_stream(ph + 16 * i);
    const uint8_t *qg = a.s4 + 1ll * row * (K >> 4) + (k_t >> 4);
    sg = ldg_stream8(qg);
    sh = ldg_stream8(qg + 8ll * (K >> 4));
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) wg[i] = wh[i] = make_uint4(0u, 0u, 0u, 0u);
  }
  // eight block scales per row -> broadcast half2
  uint32_t sgb[8], shb[8];
  {
    const uint32_t gp[4] = {cvt_e4m3x2(sg.x), cvt_e4m3x2(sg.x >> 16), cvt_e4m3x2(sg.y), cvt_e4m3x2(sg.y >> 16)};
    const uint32_t hp[4] = {cvt_e4m3x2(sh.x), cvt_e4m3x2(sh.x >> 16), cvt_e4m3x2(sh.y), cvt_e4m3x2(sh.y >> 16)};
#pragma unroll
    for (int b = 0; b < 8; ++b) {
      sgb[b] = __byte_perm(gp[b >> 1], 0u, (b & 1) ? 0x3232u : 0x1010u);
      shb[b] = __byte_perm(hp[b >> 1], 0u, (b & 1) ? 0x3232u : 0x1010u);
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint4 xq[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
      for (int j = 0; j < 4; ++j)
        xq[n][j] = (tv && xr.valid[n]) ? ld_x16(xr.row[n] + k_t + 32 * i + 8 * j) : make_uint4(0u, 0u, 0u, 0u);
    const uint32_t g4[4] = {wg[i].x, wg[i].y, wg[i].z, wg[i].w};
    const uint32_t h4[4] = {wh[i].x, wh[i].y, wh[i].z, wh[i].w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int blk = (4 * i + j) >> 1;
      uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
      cvt_e2m1x8(g4[j], a0, a1, a2, a3);
      cvt_e2m1x8(h4[j], b0, b1, b2, b3);
      a0 = hmul2_u32(a0, sgb[blk]); a1 = hmul2_u32(a1, sgb[blk]);
      a2 = hmul2_u32(a2, sgb[blk]); a3 = hmul2_u32(a3, sgb[blk]);
      b0 = hmul2_u32(b0, shb[blk]); b1 = hmul2_u32(b1, shb[blk]);
      b2 = hmul2_u32(b2, shb[blk]); b3 = hmul2_u32(b3, shb[blk]);
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        mma_16816(acc[n][0], a0, b0, a1, b1, xq[n][j].x, xq[n][j].y);
        mma_16816(acc[n][1], a2, b2, a3, b3, xq[n][j].z, xq[n][j].w);
      }
    }
  }
}

// ---- one batch of FP8: 16 rows x 256 k; this lane owns k_t .. k_t+63
template <int NT>
__device__ __forceinline__ void batch_fp8(float (&acc)[NT][2][4], const GemvArgs &a, const XRows<NT> &xr,
                                          int row, int k_t, bool tv) {
  const int K = a.K;
  uint4 wg[4], wh[4];
  if (tv) {
    const uint8_t *pg = a.w8 + 1ll * row * K + k_t;
    const uint8_t *ph = pg + 8ll * K;
#pragma unroll
    for (int i = 0; i < 4; ++i) wg[i] = ldg_stream(pg + 16 * i);
#pragma unroll
    for (int i = 0; i < 4; ++i) wh[i] = ldg_stream(ph + 16 * i);
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) wg[i] = wh[i] = make_uint4(0u, 0u, 0u, 0u);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint4 xq[NT][2];
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
      for (int j = 0; j < 2; ++j)
        xq[n][j] = (tv && xr.valid[n]) ? ld_x16(xr.row[n] + k_t + 16 * i + 8 * j) : make_uint4(0u, 0u, 0u, 0u);
    const uint32_t g4[4] = {wg[i].x, wg[i].y, wg[i].z, wg[i].w};
    const uint32_t h4[4] = {wh[i].x, wh[i].y, wh[i].z, wh[i].w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t a_lo, a_hi, b_lo, b_hi;
      cvt_e4m3x4(g4[j], a_lo, a_hi);
      cvt_e4m3x4(h4[j], b_lo, b_hi);
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        const uint4 xv = xq[n][j >> 1];
        if (j & 1) mma_16816(acc[n][1], a_lo, b_lo, a_hi, b_hi, xv.z, xv.w);
        else mma_16816(acc[n][0], a_lo, b_lo, a_hi, b_hi, xv.x, xv.y);
      }
    }
  }
}

// ---- one batch of FP16: 16 rows x 128 k; this lane owns k_t .. k_t+31
template <int NT>
__device__ __forceinline__ void batch_fp16(float (&acc)[NT][2][4], const GemvArgs &a, const XRows<NT> &xr,
                                           int row, int k_t, bool tv) {
  const int K = a.K;
  uint4 wg[4], wh[4];
  if (tv) {
    const __half *pg = a.w16 + 1ll * row * K + k_t;
    const __half *ph = pg + 8ll * K;
#pragma unroll
    for (int i = 0; i < 4; ++i) wg[i] = ldg_stream(pg + 8 * i);
#pragma unroll
    for (int i = 0; i < 4; ++i) wh[i] = ldg_stream(ph + 8 * i);
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) wg[i] = wh[i] = make_uint4(0u, 0u, 0u, 0u);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      const uint4 xv = (tv && xr.valid[n]) ? ld_x16(xr.row[n] + k_t + 8 * i) : make_uint4(0u, 0u, 0u, 0u);
      mma_16816(acc[n][0], wg[i].x, wh[i].x, wg[i].y, wh[i].y, xv.x, xv.y);
      mma_16816(acc[n][1], wg[i].z, wh[i].z, wg[i].w, wh[i].w, xv.z, xv.w);
    }
  }
}

// NT = number of 8-row activation groups (1: M <= 8, 2: M <= 16)
template <int NT>
__global__ void __maxnreg__(112) gemv_stream_kernel(GemvArgs a, int tiles4, int tiles8,
                                                                  int tiles16, int l2_prefetch_on, int status_idx) {
  constexpr int kMp = 8 * NT;                                // activation rows per slot entry
  constexpr int kSlotFloats = kMmaWarps * kTileRows * kMp;   // [warp][row][m]
  constexpr int kRing = 8 / NT;                              // flush ring depth (32 KB of slots)
  __shared__ __align__(16) float ring[kRing * kSlotFloats];
  __shared__ int meta_col[kMetaSegs * kTileRows];
  __shared__ float meta_scl[kMetaSegs * kTileRows];
  __shared__ float meta_bia[kMetaSegs * kTileRows];
  __shared__ __align__(8) uint64_t bar_full[kRing];
  __shared__ __align__(8) uint64_t bar_empty[kRing];

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int K = a.K, M = a.M;
  const int N = a.n4 + a.n8 + a.n16;

  Sched sc;
  sc.S = K / kSliceK;
  sc.t4 = tiles4;
  sc.t8 = tiles8;
  sc.e4 = tiles4 * sc.S;
  sc.e8 = sc.e4 + tiles8 * sc.S;
  sc.e16 = sc.e8 + tiles16 * sc.S;
  sc.w4 = 1ll * sc.e4 * kUnit4;
  sc.w8 = sc.w4 + 1ll * (sc.e8 - sc.e4) * kUnit8;
  sc.W = sc.w8 + 1ll * (sc.e16 - sc.e8) * kUnit16;
  sc.G = gridDim.x;
  const int s_begin = sc.boundary(blockIdx.x);
  const int s_end = sc.boundary(blockIdx.x + 1);
  const int first_tile = s_begin / sc.S;
  const int nseg = (s_end > s_begin) ? ((s_end - 1) / sc.S - first_tile + 1) : 0;
  int32_t *status = a.counters + status_idx;

  if (tid == 0) TL_MARK(0);
  if (tid == 0) {
    for (int i = 0; i < kRing; ++i) {
      mbar_init(smem_u32(&bar_full[i]), kMmaWarps);
      mbar_init(smem_u32(&bar_empty[i]), 1);
    }
    mbar_init_fence();
  }
  __syncthreads();
  // Let the next kernel in the stream become resident as early as possible; it
  // only prefetches its own weights until this grid has completed.
  pdl_launch_dependents();

  if (warp == kMmaWarps) {
    // ================================================================ epilogue warp
    if (l2_prefetch_on) {
      for (int i = 0; i < nseg; ++i) {
        const Seg sg = seg_at(sc, s_begin, s_end, first_tile + i);
        const uint8_t *base;
        long long rb;      // row pitch in bytes
        int b0, b1;        // byte range inside a row
        if (sg.fmt == 0) { base = a.w4; rb = K >> 1; b0 = sg.k0 >> 1; b1 = sg.k1 >> 1; }
        else if (sg.fmt == 1) { base = a.w8; rb = K; b0 = sg.k0; b1 = sg.k1; }
        else { base = reinterpret_cast<const uint8_t *>(a.w16); rb = 2ll * K; b0 = sg.k0 * 2; b1 = sg.k1 * 2; }
        if (sg.complete) {
          if (lane == 0) l2_prefetch(base + sg.row0 * rb, static_cast<uint32_t>(kTileRows * rb));
        } else if (lane < kTileRows) {
          l2_prefetch(base + (sg.row0 + lane) * rb + b0, static_cast<uint32_t>(b1 - b0));
        }
        if (sg.fmt == 0 && lane == 16)
          l2_prefetch(a.s4 + 1ll * sg.row0 * (K >> 4), static_cast<uint32_t>(kTileRows * (K >> 4)));
      }
    }
    // output column, scale and bias of every row this CTA finishes: constants of the
    // layer, fetched up front so that finishing a tile needs no global round trip
    if (lane < kTileRows) {
      for (int i = 0; i < nseg && i < kMetaSegs; ++i) {
        const Seg sg = seg_at(sc, s_begin, s_end, first_tile + i);
        const int prow = sg.gtile * kTileRows + lane;
        const int col = a.perm ? a.perm[prow] : prow;
        meta_col[i * kTileRows + lane] = col;
        meta_scl[i * kTileRows + lane] = (sg.fmt == 1) ? a.s8[prow - a.n4] : (sg.fmt == 0 ? a.global4 : 1.f);
        meta_bia[i * kTileRows + lane] = a.bias ? __half2float(a.bias[col]) : 0.f;
      }
    }
    __syncwarp();
    TL_MARK(1);
    pdl_wait();  // y, workspace and flags belong to this launch only after the wait
    TL_MARK(2);
    const int row = lane & 15;
    const int mh = lane >> 4;
    const int mper = (M + 1) >> 1;
    const int m_lo = mh * mper;
    const int m_hi = min(M, m_lo + mper);
    for (int q = 0; q < nseg; ++q) {
      const int idx = seg_order(q, nseg);
      const Seg sg = seg_at(sc, s_begin, s_end, first_tile + idx);
      const int slot = q % kRing;
      if (!mbar_wait(smem_u32(&bar_full[slot]), (q / kRing) & 1)) {
        if (lane == 0) atomicExch(status, 2);
        return;
      }
      const float *buf = ring + slot * kSlotFloats;
      float sum[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int m = m_lo + i;
        float v = 0.f;
        if (m < m_hi) {
#pragma unroll
          for (int w = 0; w < kMmaWarps; ++w) v += buf[(w * kTileRows + row) * kMp + m];
        }
        sum[i] = v;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_empty[slot]));

      if (!sg.starts) {
        // continuation of a tile another CTA started: publish the partial, raise the flag
        float *ws = a.workspace + 1ll * blockIdx.x * 256;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int m = m_lo + i;
          if (m < m_hi) ws[row * 16 + m] = sum[i];
        }
        __threadfence();
        __syncwarp();
        if (lane == 0) st_release_gpu(a.counters + blockIdx.x, 1);
        TL_MARK(20 + (q < 10 ? q : 10));
        continue;
      }
      if (!sg.ends) {
        // this CTA holds the first slice of a split tile: collect the other parts in CTA order
        const int b_last = sc.cta_of_slice(sg.gtile * sc.S + sc.S - 1);
        bool ok = true;
        for (int b = blockIdx.x + 1; b <= b_last && ok; ++b) {
          int seen = 0;
          if (lane == 0) {
            for (int spin = 0; spin < 2000000; ++spin) {
              if (ld_acquire_gpu(a.counters + b) != 0) { seen = 1; break; }
              __nanosleep(200);
            }
          }
          seen = __shfl_sync(0xffffffffu, seen, 0);
          if (!seen) { ok = false; break; }
          const float *pw = a.workspace + 1ll * b * 256;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int m = m_lo + i;
            if (m < m_hi) sum[i] += ld_cg_f32(pw + row * 16 + m);
          }
          __syncwarp();
          if (lane == 0) st_release_gpu(a.counters + b, 0);
        }
        if (!ok) {
          if (lane == 0) atomicExch(status, 3);
          return;
        }
      }
      {
        int col;
        float scl, bia;
        if (idx < kMetaSegs) {
          col = meta_col[idx * kTileRows + row];
          scl = meta_scl[idx * kTileRows + row];
          bia = meta_bia[idx * kTileRows + row];
        } else {
          const int prow = sg.gtile * kTileRows + row;
          col = a.perm ? a.perm[prow] : prow;
          scl = (sg.fmt == 1) ? a.s8[prow - a.n4] : (sg.fmt == 0 ? a.global4 : 1.f);
          bia = a.bias ? __half2float(a.bias[col]) : 0.f;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int m = m_lo + i;
          if (m < m_hi) a.y[1ll * m * N + col] = __float2half_rn(fmaf(sum[i], scl, bia));
        }
      }
      TL_MARK(20 + (q < 10 ? q : 10));
    }
    TL_MARK(31);
    return;
  }

  // ==================================================================== MMA warps
  const int g = lane >> 2;  // fragment row / activation row
  const int t = lane & 3;   // fragment k group

  float acc[NT][2][4];
#pragma unroll
  for (int n = 0; n < NT; ++n)
#pragma unroll
    for (int c = 0; c < 2; ++c)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[n][c][i] = 0.f;

  // x is produced by the preceding kernel: do not touch it before this.
  pdl_wait();
  if (warp == 0) TL_MARK(3);

  XRows<NT> xr;
#pragma unroll
  for (int n = 0; n < NT; ++n) {
    const int m = n * 8 + g;
    xr.valid[n] = m < M;
    xr.row[n] = a.x + 1ll * (xr.valid[n] ? m : 0) * K;
  }

  int base = 0;  // batches handed out before the current segment
  for (int q = 0; q < nseg; ++q) {
    const int idx = seg_order(q, nseg);
    const Seg sg = seg_at(sc, s_begin, s_end, first_tile + idx);
    const int first = (warp - base) & (kMmaWarps - 1);
    const int row = sg.row0 + g;
    if (sg.fmt == 0) {
      for (int j = first; j < sg.nb; j += kMmaWarps) {
        const int k_t = sg.k0 + j * 512 + t * 128;
        batch_fp4<NT>(acc, a, xr, row, k_t, k_t < sg.k1);
      }
    } else if (sg.fmt == 1) {
      for (int j = first; j < sg.nb; j += kMmaWarps) {
        const int k_t = sg.k0 + j * 256 + t * 64;
        batch_fp8<NT>(acc, a, xr, row, k_t, k_t < sg.k1);
      }
    } else {
      for (int j = first; j < sg.nb; j += kMmaWarps) {
        const int k_t = sg.k0 + j * 128 + t * 32;
        batch_fp16<NT>(acc, a, xr, row, k_t, k_t < sg.k1);
      }
    }
    base += sg.nb;
    if (warp == 0) TL_MARK(4 + (q < 14 ? q : 14));

    // ---- hand the partial sums of this segment to the epilogue warp
    const int slot = q % kRing;
    if (q >= kRing) {
      if (!mbar_wait(smem_u32(&bar_empty[slot]), ((q / kRing) - 1) & 1)) {
        if (lane == 0) atomicExch(status, 1);
        return;
      }
    }
    float *buf = ring + slot * kSlotFloats;
#pragma unroll
    for (int n = 0; n < NT; ++n) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = g + (i >> 1) * 8;
        const int m = n * 8 + 2 * t + (i & 1);
        if (m < M) buf[(warp * kTileRows + r) * kMp + m] = acc[n][0][i] + acc[n][1][i];
        acc[n][0][i] = 0.f;
        acc[n][1][i] = 0.f;
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_u32(&bar_full[slot]));
  }
}

}  // namespace

#ifdef RDQ_TIMELINE
extern "C" int rdq_debug_timeline(long long *host_out) {
  return cudaMemcpyFromSymbol(host_out, g_timeline, sizeof(long long) * 148 * 32) == cudaSuccess ? 0 : -3;
}
#endif

void gemv_stream_scratch(int N, size_t *workspace_bytes, size_t *counter_bytes) {
  const int G = sm_count();
  (void)N;
  *workspace_bytes = static_cast<size_t>(G) * 256 * sizeof(float);  // one partial tile per CTA
  *counter_bytes = (static_cast<size_t>(G) + 2) * sizeof(int32_t);  // one flag per CTA + status word
}

bool gemv_stream_supported(const GemvArgs &a) {
  if (a.M < 1 || a.M > 16) return false;
  if (a.K % kSliceK != 0) return false;
  if ((a.n4 % kTileRows) || (a.n8 % kTileRows) || (a.n16 % kTileRows)) return false;
  if (a.n4 + a.n8 + a.n16 == 0) return false;
  if (!a.workspace || !a.counters) return false;
  return true;
}

int launch_gemv_stream(const GemvArgs &a, bool pdl, bool l2_prefetch_on, cudaStream_t stream) {
  const int tiles4 = a.n4 / kTileRows, tiles8 = a.n8 / kTileRows, tiles16 = a.n16 / kTileRows;
  // Every CTA must own at least one slice: a CTA's share of the weighted slice
  // line has to be no shorter than the heaviest slice (32 units).
  const long long weight =
      1ll * (a.K / kSliceK) * (1ll * tiles4 * kUnit4 + 1ll * tiles8 * kUnit8 + 1ll * tiles16 * kUnit16);
  int G = sm_count();
  if (weight / kUnit16 < G) G = static_cast<int>(weight / kUnit16);
  if (G < 1) G = 1;

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(G));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const int pf = l2_prefetch_on ? 1 : 0;
  if (a.M <= 8) {
    RDQ_CUDA(cudaLaunchKernelEx(&cfg, gemv_stream_kernel<1>, a, tiles4, tiles8, tiles16, pf, sm_count()));
  } else {
    RDQ_CUDA(cudaLaunchKernelEx(&cfg, gemv_stream_kernel<2>, a, tiles4, tiles8, tiles16, pf, sm_count()));
  }
  return RDQ_OK;
}

}  // namespace rdq
