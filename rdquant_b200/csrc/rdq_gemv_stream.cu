// Decode GEMV (M <= 16), TMA-staged stream kernel for sm_100a.
//
// One launch streams the NVFP4, FP8 and FP16 row groups of a layer exactly once
// from HBM.  The work is cut into "slices" of 16 permuted rows x 256 k; slices
// are numbered tile-major (all k of a 16-row tile, then the next tile; NVFP4
// tiles, then FP8, then FP16) and each CTA takes one contiguous, byte-balanced
// range of them (slice weights 9 : 16 : 32 = bytes of a 16x256 slice incl.
// block scales, in units of 256 B).  Inside a CTA:
//
//   producer warp   cp.async.bulk (TMA, non-tensor) of up to 512 B per row per
//                   stage into a 9-stage shared-memory ring, mbarrier tracked;
//                   starts BEFORE griddepcontrol.wait, so under programmatic
//                   dependent launch the weights of this layer stream in while
//                   the preceding kernel is still running.
//   8 MMA warps     ldmatrix the packed bytes, convert with the hardware
//                   E2M1 / E4M3 -> f16 converters, scale NVFP4 by the block
//                   scale (exact in f16), and multiply with x on the tensor
//                   cores (mma.sync m16n8k16, weights as the 16-row operand,
//                   the M <= 8 activation rows as the 8-column operand, FP32
//                   accumulators).  Warps split the k range of a stage.
//   tile flush      per 16-row tile the 8 partial accumulators are summed
//                   through shared memory in a fixed order; FP8 channel scale
//                   and bias are applied and y[m, perm[row]] is stored.
//
// A tile whose slices are split between CTAs is finished by the last CTA to
// arrive (per-tile counter), which sums the per-CTA partials from the scratch
// workspace in CTA order, so results are bitwise reproducible.  Every wait is
// bounded; a wait that runs out sets the status word and the kernel drains.
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
constexpr int kRowPitch = 528;    // 512 B of payload + 16 B skew: conflict-free ldmatrix
constexpr int kScalePitch = 80;   // 64 B of block scales + 16 B skew
constexpr int kStageW = kTileRows * kRowPitch;                // 8448
constexpr int kStageBytes = kStageW + kTileRows * kScalePitch;  // 9728
constexpr int kStages = 9;
constexpr int kMmaWarps = 8;
constexpr int kThreads = (kMmaWarps + 1) * 32;
constexpr int kRedFloats = kMmaWarps * kTileRows * 16;  // one flush buffer: [warp][row][m]
constexpr int kSmemBytes = kStages * kStageBytes + 2 * kRedFloats * 4;  // 87552 + 16384
constexpr int kUnit4 = 9, kUnit8 = 16, kUnit16 = 32;

// Static description of the slice schedule; identical on every CTA.
struct Sched {
  int S;            // slices per tile (K / 256)
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

struct Stage {
  int fmt;    // 0 NVFP4, 1 FP8, 2 FP16
  int tile;   // tile index inside the format group
  int gtile;  // tile index over all groups
  int sl;     // first slice inside the tile
  int n;      // slices in this stage
};

__device__ __forceinline__ Stage stage_at(const Sched &sc, int s, int s_end) {
  Stage st;
  int local, cap;
  if (s < sc.e4) {
    st.fmt = 0; local = s; cap = 4;
  } else if (s < sc.e8) {
    st.fmt = 1; local = s - sc.e4; cap = 2;
  } else {
    st.fmt = 2; local = s - sc.e8; cap = 1;
  }
  st.tile = local / sc.S;
  st.sl = local - st.tile * sc.S;
  st.gtile = s / sc.S;
  int n = sc.S - st.sl;
  if (n > cap) n = cap;
  if (n > s_end - s) n = s_end - s;
  st.n = n;
  return st;
}

__device__ __forceinline__ uint4 ld_x16(const __half *p) {
  uint4 v;
  asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint2 ld_x8(const __half *p) {
  uint2 v;
  asm volatile("ld.global.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t ld_x4(const __half *p) {
  uint32_t v;
  asm volatile("ld.global.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ float ld_cg_f32(const float *p) {
  float v;
  asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p));
  return v;
}

__device__ __forceinline__ void consumer_bar() {
  asm volatile("bar.sync 1, %0;" ::"n"(kMmaWarps * 32) : "memory");
}

// NT = number of 8-row activation groups (1: M <= 8, 2: M <= 16)
template <int NT>
__global__ void __launch_bounds__(kThreads, 2) gemv_stream_kernel(GemvArgs a, int tiles4, int tiles8,
                                                                  int tiles16) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ __align__(8) uint64_t bar_full[kStages];
  __shared__ __align__(8) uint64_t bar_empty[kStages];

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int K = a.K, M = a.M;
  const int N = a.n4 + a.n8 + a.n16;

  Sched sc;
  sc.S = K / kSliceK;
  sc.e4 = tiles4 * sc.S;
  sc.e8 = sc.e4 + tiles8 * sc.S;
  sc.e16 = sc.e8 + tiles16 * sc.S;
  sc.w4 = 1ll * sc.e4 * kUnit4;
  sc.w8 = sc.w4 + 1ll * (sc.e8 - sc.e4) * kUnit8;
  sc.W = sc.w8 + 1ll * (sc.e16 - sc.e8) * kUnit16;
  sc.G = gridDim.x;
  const int s_begin = sc.boundary(blockIdx.x);
  const int s_end = sc.boundary(blockIdx.x + 1);
  int32_t *status = a.counters ? a.counters + (tiles4 + tiles8 + tiles16) : nullptr;

  if (tid == 0) {
    for (int i = 0; i < kStages; ++i) {
      mbar_init(smem_u32(&bar_full[i]), 1);
      mbar_init(smem_u32(&bar_empty[i]), kMmaWarps);
    }
    mbar_init_fence();
  }
  __syncthreads();
  // Let the next kernel in the stream become resident as early as possible; it
  // only prefetches its own weights until this grid has completed.
  pdl_launch_dependents();

  const uint32_t smem_base = smem_u32(smem);

  if (warp == kMmaWarps) {
    // ------------------------------------------------------------------ producer
    int it = 0;
    for (int s = s_begin; s < s_end; ++it) {
      const Stage st = stage_at(sc, s, s_end);
      const int slot = it % kStages;
      if (it >= kStages) {
        if (!mbar_wait(smem_u32(&bar_empty[slot]), ((it / kStages) - 1) & 1)) {
          if (status && lane == 0) atomicExch(status, 1);
          return;
        }
      }
      const uint32_t full = smem_u32(&bar_full[slot]);
      const uint32_t dst = smem_base + slot * kStageBytes;
      const int row0 = st.tile * kTileRows;
      const int k0 = st.sl * kSliceK;
      const int kel = st.n * kSliceK;
      uint32_t wbytes, sbytes = 0;
      if (st.fmt == 0) { wbytes = kel >> 1; sbytes = kel >> 4; }
      else if (st.fmt == 1) wbytes = kel;
      else wbytes = kel << 1;
      if (lane == 0) mbar_arrive_expect_tx(full, kTileRows * (wbytes + sbytes));
      __syncwarp();
      if (lane < kTileRows) {
        const int r = row0 + lane;
        const uint8_t *src;
        if (st.fmt == 0) src = a.w4 + 1ll * r * (K >> 1) + (k0 >> 1);
        else if (st.fmt == 1) src = a.w8 + 1ll * r * K + k0;
        else src = reinterpret_cast<const uint8_t *>(a.w16) + (1ll * r * K + k0) * 2;
        bulk_g2s(dst + lane * kRowPitch, src, wbytes, full);
      } else if (st.fmt == 0) {
        const int r = row0 + lane - kTileRows;
        const uint8_t *src = a.s4 + 1ll * r * (K >> 4) + (k0 >> 4);
        bulk_g2s(dst + kStageW + (lane - kTileRows) * kScalePitch, src, sbytes, full);
      }
      s += st.n;
    }
    return;
  }

  // -------------------------------------------------------------------- MMA warps
  float *red = reinterpret_cast<float *>(smem + kStages * kStageBytes);
  const int g = lane >> 2;  // fragment row / activation row
  const int t = lane & 3;   // fragment k group
  // ldmatrix source row and 16-byte column for this lane (x4: four 8x8 matrices)
  const int lm_row = (lane & 7) + ((lane >> 3) & 1) * 8;
  const int lm_sel = lane >> 4;

  float acc[NT][2][4];
#pragma unroll
  for (int n = 0; n < NT; ++n)
#pragma unroll
    for (int c = 0; c < 2; ++c)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[n][c][i] = 0.f;

  // x is produced by the preceding kernel: do not touch it (or y) before this.
  pdl_wait();

  const __half *xrow[NT];
  bool xvalid[NT];
#pragma unroll
  for (int n = 0; n < NT; ++n) {
    const int m = n * 8 + g;
    xvalid[n] = m < M;
    xrow[n] = a.x + 1ll * (xvalid[n] ? m : 0) * K;
  }

  int it = 0;
  int seg = 0;        // index of the current tile segment of this CTA
  int flush_buf = 0;
  int s = s_begin;
  bool failed = false;
  while (s < s_end) {
    const Stage st = stage_at(sc, s, s_end);
    const int slot = it % kStages;
    if (!mbar_wait(smem_u32(&bar_full[slot]), (it / kStages) & 1)) {
      if (status && lane == 0) atomicExch(status, 2);
      failed = true;
      break;
    }
    const uint32_t sbase = smem_base + slot * kStageBytes;
    const int k0 = st.sl * kSliceK;

    if (st.fmt == 0) {
      // pieces of 32 k (16 B per row); st.n pieces per warp
      const int p0 = warp * st.n;
      const uint8_t *sscale = smem + slot * kStageBytes + kStageW;
      for (int j = 0; j < st.n; j += 2) {
        const int p = p0 + j;
        const bool two = (j + 1) < st.n;
        uint32_t r0, r1, r2, r3;
        ldmatrix_x4(sbase + lm_row * kRowPitch + (p + (two ? lm_sel : 0)) * 16, r0, r1, r2, r3);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          if (h == 1 && !two) break;
          const int pp = p + h;
          const uint32_t wg = h ? r2 : r0, wg8 = h ? r3 : r1;
          // block scales: bytes (2pp, 2pp+1) of the scale row; this lane's 8 codes sit in block t>>1
          const uint32_t sraw_g = *reinterpret_cast<const uint16_t *>(sscale + g * kScalePitch + 2 * pp);
          const uint32_t sraw_g8 =
              *reinterpret_cast<const uint16_t *>(sscale + (g + 8) * kScalePitch + 2 * pp);
          const uint32_t sel = (t & 2) ? 0x3232u : 0x1010u;
          const uint32_t sg = __byte_perm(cvt_e4m3x2(sraw_g), 0u, sel);
          const uint32_t sg8 = __byte_perm(cvt_e4m3x2(sraw_g8), 0u, sel);
          uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
          cvt_e2m1x8(wg, a0, a1, a2, a3);
          cvt_e2m1x8(wg8, b0, b1, b2, b3);
          a0 = hmul2_u32(a0, sg); a1 = hmul2_u32(a1, sg); a2 = hmul2_u32(a2, sg); a3 = hmul2_u32(a3, sg);
          b0 = hmul2_u32(b0, sg8); b1 = hmul2_u32(b1, sg8); b2 = hmul2_u32(b2, sg8); b3 = hmul2_u32(b3, sg8);
          const int kk = k0 + pp * 32 + t * 8;
#pragma unroll
          for (int n = 0; n < NT; ++n) {
            uint4 xv = make_uint4(0u, 0u, 0u, 0u);
            if (xvalid[n]) xv = ld_x16(xrow[n] + kk);
            mma_16816(acc[n][0], a0, b0, a1, b1, xv.x, xv.y);
            mma_16816(acc[n][1], a2, b2, a3, b3, xv.z, xv.w);
          }
        }
      }
    } else if (st.fmt == 1) {
      // pieces of 16 k (16 B per row); 2*st.n pieces per warp
      const int p0 = warp * 2 * st.n;
      for (int j = 0; j < 2 * st.n; j += 2) {
        const int p = p0 + j;
        uint32_t r0, r1, r2, r3;
        ldmatrix_x4(sbase + lm_row * kRowPitch + (p + lm_sel) * 16, r0, r1, r2, r3);
        uint32_t a0, a4, a2, a6, c0, c4, c2, c6;
        cvt_e4m3x4(r0, a0, a4);
        cvt_e4m3x4(r1, a2, a6);
        cvt_e4m3x4(r2, c0, c4);
        cvt_e4m3x4(r3, c2, c6);
        const int kk = k0 + p * 16 + t * 4;
#pragma unroll
        for (int n = 0; n < NT; ++n) {
          uint2 x0 = make_uint2(0u, 0u), x1 = make_uint2(0u, 0u);
          if (xvalid[n]) {
            x0 = ld_x8(xrow[n] + kk);
            x1 = ld_x8(xrow[n] + kk + 16);
          }
          mma_16816(acc[n][0], a0, a2, a4, a6, x0.x, x0.y);
          mma_16816(acc[n][1], c0, c2, c4, c6, x1.x, x1.y);
        }
      }
    } else {
      // FP16: pieces of 16 k (32 B per row); 16 pieces per slice, 2 per warp
      const int p0 = warp * 2 * st.n;
      for (int j = 0; j < 2 * st.n; ++j) {
        const int p = p0 + j;
        uint32_t r0, r1, r2, r3;
        ldmatrix_x4(sbase + lm_row * kRowPitch + p * 32 + lm_sel * 16, r0, r1, r2, r3);
        const int kk = k0 + p * 16 + t * 2;
#pragma unroll
        for (int n = 0; n < NT; ++n) {
          uint32_t x0 = 0u, x1 = 0u;
          if (xvalid[n]) {
            x0 = ld_x4(xrow[n] + kk);
            x1 = ld_x4(xrow[n] + kk + 8);
          }
          mma_16816(acc[n][j & 1], r0, r1, r2, r3, x0, x1);
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_u32(&bar_empty[slot]));
    ++it;
    s += st.n;

    // ---- tile flush when the tile (or this CTA's range) ends
    const bool tile_done = (st.sl + st.n == sc.S);
    if (tile_done || s >= s_end) {
      float *buf = red + flush_buf * kRedFloats;
#pragma unroll
      for (int n = 0; n < NT; ++n) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int row = g + (i >> 1) * 8;
          const int m = n * 8 + 2 * t + (i & 1);
          if (m < M) buf[(warp * kTileRows + row) * 16 + m] = acc[n][0][i] + acc[n][1][i];
          acc[n][0][i] = 0.f;
          acc[n][1][i] = 0.f;
        }
      }
      consumer_bar();
      if (warp == (seg & (kMmaWarps - 1))) {
        // this warp finishes the tile: lane -> (row, half of the m range)
        const int row = lane & 15;
        const int mh = lane >> 4;
        const int mper = (M + 1) >> 1;
        const int m_lo = mh * mper;
        const int m_hi = min(M, m_lo + mper);
        float sum[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) sum[i] = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int m = m_lo + i;
          if (m < m_hi) {
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < kMmaWarps; ++w) v += buf[(w * kTileRows + row) * 16 + m];
            sum[i] = v;
          }
        }
        // segment coverage of the tile
        const int tile_first_slice = st.gtile * sc.S;
        const int seg_first = max(s_begin, tile_first_slice);
        const bool complete = (seg_first == tile_first_slice) && tile_done;
        bool finalize = complete;
        if (!complete) {
          // split tile: publish the partial, last arriver sums all parts in CTA order
          const int myslot = (seg == 0) ? 0 : 1;
          float *ws = a.workspace + (1ll * (blockIdx.x * 2 + myslot)) * 256;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int m = m_lo + i;
            if (m < m_hi) ws[row * 16 + m] = sum[i];
          }
          __threadfence();
          __syncwarp();
          int old = 0;
          const int b_first = sc.cta_of_slice(tile_first_slice);
          const int b_last = sc.cta_of_slice(tile_first_slice + sc.S - 1);
          if (lane == 0) old = atomicAdd(a.counters + st.gtile, 1);
          old = __shfl_sync(0xffffffffu, old, 0);
          if (old == b_last - b_first) {
            __threadfence();
#pragma unroll
            for (int i = 0; i < 8; ++i) sum[i] = 0.f;
            for (int b = b_first; b <= b_last; ++b) {
              const int bslot = (sc.boundary(b) >= tile_first_slice) ? 0 : 1;
              const float *pw = a.workspace + (1ll * (b * 2 + bslot)) * 256;
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const int m = m_lo + i;
                if (m < m_hi) sum[i] += ld_cg_f32(pw + row * 16 + m);
              }
            }
            if (lane == 0) atomicExch(a.counters + st.gtile, 0);
            finalize = true;
          }
        }
        if (finalize) {
          const int prow = st.gtile * kTileRows + row;  // permuted row index over all groups
          const int col = a.perm ? a.perm[prow] : prow;
          const float scl = (st.fmt == 1) ? a.s8[prow - a.n4] : (st.fmt == 0 ? a.global4 : 1.f);
          const float bia = a.bias ? __half2float(a.bias[col]) : 0.f;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int m = m_lo + i;
            if (m < m_hi) a.y[1ll * m * N + col] = __float2half_rn(fmaf(sum[i], scl, bia));
          }
        }
      }
      flush_buf ^= 1;
      ++seg;
    }
  }
  (void)failed;
}

}  // namespace

void gemv_stream_scratch(int N, size_t *workspace_bytes, size_t *counter_bytes) {
  const int G = sm_count();
  *workspace_bytes = static_cast<size_t>(G) * 2 * 256 * sizeof(float);
  *counter_bytes = (static_cast<size_t>(N / kTileRows) + 2) * sizeof(int32_t);
}

bool gemv_stream_supported(const GemvArgs &a) {
  if (a.M < 1 || a.M > 16) return false;
  if (a.K % kSliceK != 0) return false;
  if ((a.n4 % kTileRows) || (a.n8 % kTileRows) || (a.n16 % kTileRows)) return false;
  if (a.n4 + a.n8 + a.n16 == 0) return false;
  if (!a.workspace || !a.counters) return false;
  return true;
}

int launch_gemv_stream(const GemvArgs &a, bool pdl, cudaStream_t stream) {
  static bool attr_set[64] = {};
  int dev = 0;
  RDQ_CUDA(cudaGetDevice(&dev));
  if (dev < 64 && !attr_set[dev]) {
    RDQ_CUDA(cudaFuncSetAttribute(gemv_stream_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  kSmemBytes));
    RDQ_CUDA(cudaFuncSetAttribute(gemv_stream_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  kSmemBytes));
    attr_set[dev] = true;
  }
  const int tiles4 = a.n4 / kTileRows, tiles8 = a.n8 / kTileRows, tiles16 = a.n16 / kTileRows;
  const long long slices = 1ll * (tiles4 + tiles8 + tiles16) * (a.K / kSliceK);
  // Every CTA must own at least one slice: a CTA's share of the weighted slice
  // line has to be no shorter than the heaviest slice (32 units).
  const long long weight = 1ll * (a.K / kSliceK) * (1ll * tiles4 * kUnit4 + 1ll * tiles8 * kUnit8 + 1ll * tiles16 * kUnit16);
  int G = sm_count();
  if (weight / kUnit16 < G) G = static_cast<int>(weight / kUnit16);
  if (G < 1) G = 1;
  (void)slices;

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(G));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (a.M <= 8) {
    RDQ_CUDA(cudaLaunchKernelEx(&cfg, gemv_stream_kernel<1>, a, tiles4, tiles8, tiles16));
  } else {
    RDQ_CUDA(cudaLaunchKernelEx(&cfg, gemv_stream_kernel<2>, a, tiles4, tiles8, tiles16));
  }
  return RDQ_OK;
}

}  // namespace rdq
