// Kernel and launcher of rdq_gemm.cu (included at its end; see the header comment there).
namespace rdq {

namespace {

// Status word of the GEMM on this device: 0, or 1 once a CTA gave up a bounded wait (2: the
// time-out self-test).  Read and cleared by gemm_status().
__device__ int g_gemm_status;


__device__ __forceinline__ uint32_t ldg_nc2(const void *p) {
  uint16_t v;
  asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(v) : "l"(p));
  return v;
}

// Stage bookkeeping of one producer thread: before writing stage s of round ph it waits until
// the MMA has released it; afterwards it makes its generic-proxy writes visible to the async
// proxy and arrives on full[s].
template <int NS>
struct StageCursor {
  int s = 0, ph = 0;
  bool alive = true;
  __device__ __forceinline__ void begin(GemmSmem &S) {
    if (ph > 0 && alive) alive = gemm_wait(&S.empty[s], (ph - 1) & 1, &S.abort_flag);
  }
  // every lane fences its own writes; one arrival per warp (hundreds of arrivals per stage on
  // one barrier were the slowest part of a k block)
  __device__ __forceinline__ void end(GemmSmem &S) {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncwarp();
    if ((threadIdx.x & 31) == 0) mbar_arrive(smem_u32(&S.full[s]));
    if (++s == NS) { s = 0; ++ph; }
  }
};

// ---- dequantisation: eight lanes share one weight row of the tile, one 16-byte chunk (8 k)
// each, so that a quarter warp writes the 128 contiguous (swizzled) bytes of a row and reads
// 32 / 64 / 128 contiguous packed bytes.  The tile's rows are sorted by format and padded to
// groups of four (one group per warp and step); a warp takes every W-th group.
__device__ __forceinline__ uint32_t ldg_nc1(const void *p) {
  uint32_t v;
  asm volatile("ld.global.nc.u8 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ uint2 ldg_nc8(const void *p) {
  uint2 v;
  asm volatile("ld.global.nc.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}

template <int NS, int SB, int TMAX, int PF>
__device__ __forceinline__ void produce_rows(GemmSmem &S, const GemmArgs &a, uint32_t b_base, int pwarp, int nwarps,
                                             int lane, int kb0, int nkb) {
  const int chunk = lane & 7, sub = lane >> 3;
  const int nq = S.nquad;
  // per task: 32-bit byte offset of this lane's chunk from the format's weight tensor (the
  // launcher checks that the tensors are below 4 GB), offset of its block scale (NVFP4), row
  // offset inside a stage (swizzle applied), format (3 = write zeros, 4 = nothing to do)
  uint32_t woff[TMAX], soff[TMAX], roff[TMAX];
  int fmt[TMAX];
#pragma unroll
  for (int t = 0; t < TMAX; ++t) {
    const int quad = pwarp + t * nwarps;
    fmt[t] = 4;
    woff[t] = 0;
    soff[t] = 0;
    roff[t] = 0;
    if (quad < nq) {
      const int j = S.prow[quad * 4 + sub];
      if (j >= 0) {
        const int r = S.row_perm[j];
        roff[t] = (j >> 3) * 1024 + (j & 7) * 128 + ((chunk ^ (j & 7)) << 4);
        if (r < 0) {
          fmt[t] = 3;
        } else if (r < a.n4) {
          fmt[t] = 0;
          woff[t] = static_cast<uint32_t>(r) * (a.K >> 1) + chunk * 4;
          soff[t] = static_cast<uint32_t>(r) * (a.K >> 4) + (chunk >> 1);
        } else if (r < a.n4 + a.n8) {
          fmt[t] = 1;
          woff[t] = static_cast<uint32_t>(r - a.n4) * a.K + chunk * 8;
        } else {
          fmt[t] = 2;
          woff[t] = static_cast<uint32_t>(r - a.n4 - a.n8) * (a.K * 2) + chunk * 16;
        }
      }
    }
  }
  const uint8_t *w16b = reinterpret_cast<const uint8_t *>(a.w16);
  auto load = [&](int t, int kb) {
    uint4 d = make_uint4(0u, 0u, 0u, 0u);
    if (fmt[t] == 0) {
      d.x = ldg_nc4(a.w4 + (woff[t] + kb * 32u));
      d.y = ldg_nc1(a.s4 + (soff[t] + kb * 4u));
    } else if (fmt[t] == 1) {
      const uint2 v = ldg_nc8(a.w8 + (woff[t] + kb * 64u));
      d.x = v.x;
      d.y = v.y;
    } else if (fmt[t] == 2) {
      d = ldg_nc16(w16b + (woff[t] + kb * 128u));
    }
    return d;
  };
  StageCursor<NS> cur;
  // packed bytes of the next PF k blocks sit in registers: a load is issued PF blocks before
  // its use (L2 latency under load is longer than one k block's MMA time)
  uint4 q[PF][TMAX];
#pragma unroll
  for (int p = 0; p < PF; ++p) {
#pragma unroll
    for (int t = 0; t < TMAX; ++t) q[p][t] = (kb0 + p < nkb) ? load(t, kb0 + p) : make_uint4(0u, 0u, 0u, 0u);
  }
  for (int kbase = kb0; kbase < nkb; kbase += PF) {
#pragma unroll
    for (int p = 0; p < PF; ++p) {
      const int kb = kbase + p;
      if (kb >= nkb) break;
      cur.begin(S);
      const uint32_t sbase = b_base + cur.s * SB;
      // convert straight out of the prefetch registers, then refill them for k block kb + PF
#pragma unroll
      for (int t = 0; t < TMAX; ++t) {
        const uint4 c = q[p][t];
        uint32_t o0 = 0u, o1 = 0u, o2 = 0u, o3 = 0u;
        if (fmt[t] == 0) {
          const uint32_t scl = __byte_perm(cvt_e4m3x2(c.y), 0u, 0x1010u);
          cvt_e2m1x8(c.x, o0, o1, o2, o3);
          o0 = hmul2_u32(o0, scl);
          o1 = hmul2_u32(o1, scl);
          o2 = hmul2_u32(o2, scl);
          o3 = hmul2_u32(o3, scl);
        } else if (fmt[t] == 1) {
          cvt_e4m3x4(c.x, o0, o1);
          cvt_e4m3x4(c.y, o2, o3);
        } else if (fmt[t] == 2) {
          o0 = c.x; o1 = c.y; o2 = c.z; o3 = c.w;
        }
        if (fmt[t] != 4)
          asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(sbase + roff[t]), "r"(o0), "r"(o1), "r"(o2), "r"(o3)
                       : "memory");
        if (kb + PF < nkb) q[p][t] = load(t, kb + PF);
      }
      cur.end(S);
    }
  }
}

template <int MT, int BN>
__global__ void __launch_bounds__(GemmCfg<MT, BN>::kThreads, 1)
gemm_mixed_kernel(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ GemmArgs a) {
  using Cfg = GemmCfg<MT, BN>;
  constexpr int NS = Cfg::kStages, SB = Cfg::kStageB;
  constexpr int kStageAll = Cfg::kStageAll;
  constexpr uint32_t kCols = Cfg::kTmemCols;
  extern __shared__ uint8_t smem_raw[];
  __shared__ GemmSmem S;
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t a_base = (raw_addr + 1023u) & ~1023u;  // swizzled tiles need 1024-byte alignment
  const uint32_t b_base = a_base + NS * kStageAll;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int m0 = blockIdx.x * BM * MT;
  const int n0 = blockIdx.y * BN;
  const int N = a.n4 + a.n8 + a.n16;
  // this CTA's k blocks [kb0, nkb): the whole K, or one of ksplit equal parts (blockIdx.z)
  const int nkb_all = a.K / BK;
  const int kb0 = static_cast<int>(1ll * blockIdx.z * nkb_all / a.ksplit);
  const int nkb = static_cast<int>(1ll * (blockIdx.z + 1) * nkb_all / a.ksplit);

  if (tid == 32) {
    // the TMA unit reads the tensor map from memory: start that fetch now
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&xmap)) : "memory");
  }
  if (tid == 0) {
    for (int i = 0; i < NS; ++i) {
      mbar_init(smem_u32(&S.full[i]), Cfg::kProducerWarps + 1);  // producer warps + the TMA thread
      mbar_init(smem_u32(&S.empty[i]), 1);
    }
    mbar_init(smem_u32(&S.accum), 1);
    mbar_init(smem_u32(&S.never), 1);
    S.abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&S.tmem_base)),
                 "r"(kCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  for (int j = tid - 64; j >= 0 && j < BN; j += Cfg::kProducers) {
    const int n = n0 + j;
    int r = -1;
    float scl = 0.f, bia = 0.f;
    if (n < N) {
      r = a.inv_perm ? a.inv_perm[n] : n;
      scl = (r < a.n4) ? a.global4 : (r < a.n4 + a.n8 ? a.s8[r - a.n4] : 1.f);
      bia = a.bias ? __half2float(a.bias[n]) : 0.f;
    }
    S.row_perm[j] = r;
    S.colscale[j] = scl;
    S.colbias[j] = bia;
  }
  __syncthreads();
  if (warp == 2) {
    // sort the tile rows by format (stable); each format's rows are padded to groups of four
    int base = 0;
#pragma unroll 1
    for (int ff = 0; ff < 3; ++ff) {
      int cnt = 0;
      for (int round = 0; round < BN / 32; ++round) {
        const int j = round * 32 + lane;
        const int r = S.row_perm[j];
        const int f = (r >= 0 && r < a.n4) ? 0 : ((r >= a.n4 && r < a.n4 + a.n8) ? 1 : 2);
        const uint32_t mask = __ballot_sync(0xffffffffu, f == ff);
        if (f == ff) S.prow[base + cnt + __popc(mask & ((1u << lane) - 1u))] = j;
        cnt += __popc(mask);
      }
      const int padded = (cnt + 3) & ~3;
      if (lane < padded - cnt) S.prow[base + cnt + lane] = -1;
      base += padded;
    }
    if (lane == 0) S.nquad = base >> 2;
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = S.tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------- activation loads (TMA)
    if (lane == 0) {
      bool alive = true;
      int s = 0, ph = 0;
      for (int kb = kb0; kb < nkb && alive; ++kb) {
        if (ph > 0) alive = gemm_wait(&S.empty[s], (ph - 1) & 1, &S.abort_flag);
        if (!alive) break;
        const uint32_t full = smem_u32(&S.full[s]);
        mbar_arrive_expect_tx(full, kStageAll);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
          tma_load_2d(a_base + s * kStageAll + mt * kStageA, &xmap, kb * BK, m0 + mt * BM, full);
        if (++s == NS) { s = 0; ++ph; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------------ MMA issue
    if (lane == 0) {
      constexpr uint32_t idesc = (1u << 4) | (static_cast<uint32_t>(BN >> 3) << 17) | (static_cast<uint32_t>(BM >> 4) << 24);
      bool alive = true;
      int s = 0, ph = 0;
      for (int kb = kb0; kb < nkb && alive; ++kb) {
        alive = gemm_wait(&S.full[s], ph & 1, &S.abort_flag);
        if (!alive) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint64_t db = make_desc_sw128(b_base + s * SB);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          const uint64_t da = make_desc_sw128(a_base + s * kStageAll + mt * kStageA);
#pragma unroll
          for (int k4 = 0; k4 < BK / 16; ++k4)
            umma_f16(tmem + mt * BN, da + 2 * k4, db + 2 * k4, idesc, (kb != kb0 || k4 != 0) ? 1u : 0u);
        }
        umma_commit(smem_u32(&S.empty[s]));
        if (++s == NS) { s = 0; ++ph; }
      }
      umma_commit(smem_u32(&S.accum));
    }
  } else {
    // ------------------------------------------------------------- weight dequantisation
    produce_rows<NS, SB, Cfg::kTasks, Cfg::kPrefetch>(S, a, b_base, warp - 2, Cfg::kProducerWarps, lane, kb0, nkb);

    // ----------------------------------------------------------------------- epilogue
    // A warp may read the tensor-memory lanes 32 (warp % 4) ...; the producer warps that share a
    // lane quarter take the 32-column chunks of the accumulators in turn.
    constexpr int kEpiWarps = (Cfg::kProducerWarps / 4) * 4;  // whole sets of four warps
    constexpr int kEpiPitch = 144;  // staging row pitch in bytes: 128 B payload, odd multiple of 16 B
    if (warp - 2 < kEpiWarps) {
      const bool ok = gemm_wait(&S.accum, 0, &S.abort_flag);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int q = warp & 3;  // tensor-memory lane quarter this warp may read
      const int sub = (warp - 2) >> 2;
      if (ok) {
#pragma unroll 1
        // a warp takes pairs of adjacent 32-channel chunks: 64 channels = 128 B of an output row
        for (int cp = sub; cp < MT * (BN / 64); cp += kEpiWarps / 4) {
          const int mt = cp / (BN / 64);
          const int m = m0 + mt * BM + q * 32 + lane;
          const bool wide = a.ksplit == 1 && n0 + (cp % (BN / 64)) * 64 + 64 <= N && (N & 7) == 0;
          const uint32_t stg = a_base + static_cast<uint32_t>(warp - 2) * (32 * kEpiPitch);
#pragma unroll 1
          for (int hh = 0; hh < 2; ++hh) {
          const int cc = (cp % (BN / 64)) * 2 + hh;
          uint32_t r[32];
          tmem_ld32(tmem + (static_cast<uint32_t>(q * 32) << 16) + mt * BN + cc * 32, r);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          if (m < a.M && a.ksplit > 1) {
            // split k range: raw FP32 sums go to this part's plane; scale, bias and the f16
            // conversion happen in the reduction kernel
            float *dst = a.partial + (1ll * blockIdx.z * a.M + m) * N + n0 + cc * 32;
            if (n0 + cc * 32 + 32 <= N && (N & 3) == 0) {
#pragma unroll
              for (int v = 0; v < 8; ++v)
                *reinterpret_cast<uint4 *>(dst + 4 * v) = make_uint4(r[4 * v], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]);
            } else {
              for (int e = 0; e < 32; ++e)
                if (n0 + cc * 32 + e < N) dst[e] = __uint_as_float(r[e]);
            }
          } else if (wide) {
            // Whole 64-channel pair: the warp turns its 32 rows x 128 B around in shared memory
            // (the stage buffers are free once the accumulators are complete) so that a store
            // instruction writes four rows x 128 contiguous bytes instead of 32 rows x 16 B:
            // the stores of a tile otherwise take three times as long as the rest of its epilogue.
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint32_t o[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int c = cc * 32 + v * 8 + e * 2;
                const float f0 = fmaf(__uint_as_float(r[v * 8 + e * 2]), S.colscale[c], S.colbias[c]);
                const float f1 = fmaf(__uint_as_float(r[v * 8 + e * 2 + 1]), S.colscale[c + 1], S.colbias[c + 1]);
                const __half2 h = __floats2half2_rn(f0, f1);
                o[e] = *reinterpret_cast<const uint32_t *>(&h);
              }
              asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(stg + lane * kEpiPitch + hh * 64 + v * 16), "r"(o[0]),
                           "r"(o[1]), "r"(o[2]), "r"(o[3])
                           : "memory");
            }
          } else if (m < a.M) {
            __half *dst = a.y + 1ll * m * N + n0 + cc * 32;
            for (int e = 0; e < 32; ++e) {
              const int c = cc * 32 + e;
              if (n0 + c < N) dst[e] = __float2half_rn(fmaf(__uint_as_float(r[e]), S.colscale[c], S.colbias[c]));
            }
          }
          }  // hh
          if (wide) {
            __syncwarp();
            const int m_base = m0 + mt * BM + q * 32;
            const int c0 = (cp % (BN / 64)) * 64;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int row = i * 4 + (lane >> 3), piece = lane & 7;
              uint4 val;
              asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                           : "=r"(val.x), "=r"(val.y), "=r"(val.z), "=r"(val.w)
                           : "r"(stg + row * kEpiPitch + piece * 16)
                           : "memory");
              if (m_base + row < a.M) *reinterpret_cast<uint4 *>(a.y + 1ll * (m_base + row) * N + n0 + c0 + piece * 8) = val;
            }
            __syncwarp();
          }
        }
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kCols)
                 : "memory");
  }
  if (tid == 0 && S.abort_flag) atomicExch(&g_gemm_status, 1);
  if (a.test_timeout && tid == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) {
    // Self-test of the time-out path: the tile is finished and nothing of this CTA is in flight;
    // wait (three suspended tries) on a barrier that nothing completes and report it.
    if (!mbar_wait(smem_u32(&S.never), 0, 3u)) atomicExch(&g_gemm_status, 2);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// y = f16(sum over parts * channel scale + bias) for a split launch
__global__ void __launch_bounds__(256) gemm_reduce_kernel(const GemmArgs a, int N) {
  const long long total = 1ll * a.M * N;
  for (long long i = 1ll * blockIdx.x * blockDim.x + threadIdx.x; i < total; i += 1ll * gridDim.x * blockDim.x) {
    const int n = static_cast<int>(i % N);
    float v = 0.f;
    for (int z = 0; z < a.ksplit; ++z) v += a.partial[z * total + i];
    const int r = a.inv_perm ? a.inv_perm[n] : n;
    const float scl = (r < a.n4) ? a.global4 : (r < a.n4 + a.n8 ? a.s8[r - a.n4] : 1.f);
    const float bia = a.bias ? __half2float(a.bias[n]) : 0.f;
    a.y[i] = __float2half_rn(fmaf(v, scl, bia));
  }
}

template <int MT, int BN>
int launch_cfg(const CUtensorMap &xmap, const GemmArgs &a, int N, cudaStream_t stream) {
  using Cfg = GemmCfg<MT, BN>;
  static std::atomic<bool> attr_done[64];
  int dev = 0;
  RDQ_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || !attr_done[dev].load()) {
    RDQ_CUDA(cudaFuncSetAttribute(gemm_mixed_kernel<MT, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmem));
    if (dev >= 0 && dev < 64) attr_done[dev].store(true);
  }
  const dim3 grid((a.M + MT * BM - 1) / (MT * BM), (N + BN - 1) / BN, a.ksplit);
  gemm_mixed_kernel<MT, BN><<<grid, Cfg::kThreads, Cfg::kSmem, stream>>>(xmap, a);
  RDQ_CUDA(cudaGetLastError());
  if (a.ksplit > 1) {
    long long blocks = (1ll * a.M * N + 255) / 256;
    if (blocks > 8ll * sm_count()) blocks = 8ll * sm_count();
    gemm_reduce_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(a, N);
    RDQ_CUDA(cudaGetLastError());
  }
  return RDQ_OK;
}

}  // namespace

namespace {
// Tile configuration (0: 128 x 128, 1: 256 tokens x 128, 2: 256 x 256) and k split of a problem,
// chosen by a small time estimate: waves of CTAs x work per CTA / efficiency of the
// configuration.  Efficiencies are the measured throughputs of the three configurations on
// large problems (424 / 715 / 921 TFLOP/s): wider tiles convert each weight byte for more
// tokens.  Few tiles leave SMs idle for the whole launch: then up to four CTAs share a tile's
// k range (as long as each keeps at least eight k blocks) and a second kernel adds their sums.
struct GemmPlan {
  int cfg, ksplit;
};
GemmPlan gemm_plan(int M, int N, int K) {
  const int sms = sm_count();
  const int nkb = K / BK;
  const long long t256 = (M + 255) / 256, t128 = (M + 127) / 128;
  const long long n256 = (N + 255) / 256, n128 = (N + 127) / 128;
  const long long tiles[3] = {t128 * n128, t256 * n128, t256 * n256};
  const double area[3] = {128.0 * 128, 256.0 * 128, 256.0 * 256};
  const double eff[3] = {0.46, 0.78, 1.0};
  GemmPlan best{0, 1};
  double best_t = 0;
  for (int c = 0; c < 3; ++c) {
    int split = 1;
    if (tiles[c] * 2 <= sms) {
      split = static_cast<int>(sms / tiles[c]);
      if (split > 4) split = 4;
      if (split > nkb / 8) split = nkb / 8;
      if (split < 1) split = 1;
    }
    const long long waves = (tiles[c] * split + sms - 1) / sms;
    const double t = waves * area[c] / eff[c] / split * (split > 1 ? 1.15 : 1.0);
    if (c == 0 || t < best_t) {
      best_t = t;
      best = GemmPlan{c, split};
    }
  }
  return best;
}
}  // namespace


namespace {
std::atomic<int> g_gemm_test_timeout{0};
}

void gemm_set_test_timeout(bool on) { g_gemm_test_timeout.store(on ? 1 : 0); }

int gemm_status(bool reset, cudaStream_t stream) {
  int code = 0;
  RDQ_CUDA(cudaMemcpyFromSymbolAsync(&code, g_gemm_status, sizeof(code), 0, cudaMemcpyDeviceToHost, stream));
  RDQ_CUDA(cudaStreamSynchronize(stream));
  if (reset && code != 0) {
    const int zero = 0;
    RDQ_CUDA(cudaMemcpyToSymbolAsync(g_gemm_status, &zero, sizeof(zero), 0, cudaMemcpyHostToDevice, stream));
    RDQ_CUDA(cudaStreamSynchronize(stream));
  }
  RDQ_REQUIRE(code == 0, RDQ_E_DEVICE, "prefill GEMM: a bounded device-side wait ran out (status %d%s); results of that launch are invalid",
              code, code == 2 ? ": time-out self-test" : "");
  return RDQ_OK;
}

int launch_gemm(const GemmArgs &a, void *workspace, size_t workspace_bytes, cudaStream_t stream) {
  static std::atomic<EncodeTiledFn> encode_cached{nullptr};
  EncodeTiledFn encode = encode_cached.load();
  if (!encode) {
    cudaDriverEntryPointQueryResult qr;
    void *fn = nullptr;
    RDQ_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qr));
    RDQ_REQUIRE(fn != nullptr && qr == cudaDriverEntryPointSuccess, RDQ_E_CUDA, "cuTensorMapEncodeTiled is not available");
    encode = reinterpret_cast<EncodeTiledFn>(fn);
    encode_cached.store(encode);
  }
  const int N = a.n4 + a.n8 + a.n16;
  CUtensorMap xmap;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(a.K), static_cast<cuuint64_t>(a.M)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(a.K) * 2};
  const cuuint32_t box[2] = {BK, BM};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult rc = encode(&xmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half *>(a.x), dims, strides, box, estr,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  RDQ_REQUIRE(rc == CUDA_SUCCESS, RDQ_E_CUDA, "cuTensorMapEncodeTiled failed with code %d", static_cast<int>(rc));
  // the largest tile that still gives every SM a CTA: 256 tokens x 256 channels, 256 x 128, 128 x 128
  GemmArgs b = a;
  const GemmPlan plan = gemm_plan(a.M, N, a.K);
  b.ksplit = 1;
  b.partial = nullptr;
  b.test_timeout = g_gemm_test_timeout.load();
  if (plan.ksplit > 1 && workspace != nullptr && workspace_bytes >= sizeof(float) * plan.ksplit * a.M * N) {
    b.ksplit = plan.ksplit;
    b.partial = static_cast<float *>(workspace);
  }
  if (plan.cfg == 2) return launch_cfg<2, 256>(xmap, b, N, stream);
  if (plan.cfg == 1) return launch_cfg<2, 128>(xmap, b, N, stream);
  return launch_cfg<1, 128>(xmap, b, N, stream);
}

size_t gemm_workspace_bytes(int M, int N, int K) {
  const GemmPlan plan = gemm_plan(M, N, K);
  return plan.ksplit > 1 ? sizeof(float) * plan.ksplit * M * N : 0;
}

}  // namespace rdq
