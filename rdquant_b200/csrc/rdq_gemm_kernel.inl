// Kernel and launcher of rdq_gemm.cu (included at its end; see the header comment there).
namespace rdq {

namespace {

__device__ int g_gemm_aborts;  // launches that hit a bounded-wait timeout (diagnostic counter)

// ---- dequantisation loops: one thread = one weight row of the tile, all k blocks --------
// Common stage protocol: wait until the MMA has released stage s, write the row, make the
// generic-proxy writes visible to the async proxy, arrive on full[s].
#define RDQ_STAGE_BEGIN(kb)                                                         \
  const int s = (kb) & (kStages - 1);                                               \
  if ((kb) >= kStages && alive) alive = gemm_wait(&S.empty[s], (((kb) / kStages) - 1) & 1, &S.abort_flag); \
  const uint32_t row_base = b_base + s * kStageB + row_off;
#define RDQ_STAGE_END()                                                             \
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");                      \
  mbar_arrive(smem_u32(&S.full[s]));

// A thread owns HALF a weight row of the tile (32 of the 64 k of a block: chunks 4h .. 4h+3).
__device__ __forceinline__ uint32_t ldg_nc2(const void *p) {
  uint16_t v;
  asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(v) : "l"(p));
  return v;
}

__device__ __forceinline__ void produce_fp4(GemmSmem &S, const GemmArgs &a, uint32_t b_base, int j, int h, int r, int nkb) {
  const uint32_t row_off = (j >> 3) * 1024 + (j & 7) * 128;
  const int sw = j & 7;
  const uint8_t *wp = a.w4 + 1ll * r * (a.K >> 1) + h * 16;
  const uint8_t *sp = a.s4 + 1ll * r * (a.K >> 4) + h * 2;
  bool alive = true;
  uint4 q0 = ldg_nc16(wp);
  uint32_t sc = ldg_nc2(sp);
  for (int kb = 0; kb < nkb; ++kb) {
    const uint4 c0 = q0;
    const uint32_t csc = sc;
    if (kb + 1 < nkb) {
      q0 = ldg_nc16(wp + (kb + 1) * 32);
      sc = ldg_nc2(sp + (kb + 1) * 4);
    }
    RDQ_STAGE_BEGIN(kb)
    const uint32_t s01 = cvt_e4m3x2(csc);
    const uint32_t sb[2] = {__byte_perm(s01, 0u, 0x1010u), __byte_perm(s01, 0u, 0x3232u)};
    const uint32_t w[4] = {c0.x, c0.y, c0.z, c0.w};
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t h0, h1, h2, h3;
      cvt_e2m1x8(w[c], h0, h1, h2, h3);
      const uint32_t scl = sb[c >> 1];
      st_chunk(row_base, sw, 4 * h + c, hmul2_u32(h0, scl), hmul2_u32(h1, scl), hmul2_u32(h2, scl), hmul2_u32(h3, scl));
    }
    RDQ_STAGE_END()
  }
}

__device__ __forceinline__ void produce_fp8(GemmSmem &S, const GemmArgs &a, uint32_t b_base, int j, int h, int r, int nkb) {
  const uint32_t row_off = (j >> 3) * 1024 + (j & 7) * 128;
  const int sw = j & 7;
  const uint8_t *wp = a.w8 + 1ll * (r - a.n4) * a.K + h * 32;
  bool alive = true;
  uint4 q[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) q[i] = ldg_nc16(wp + 16 * i);
  for (int kb = 0; kb < nkb; ++kb) {
    uint4 c[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) c[i] = q[i];
    if (kb + 1 < nkb) {
#pragma unroll
      for (int i = 0; i < 2; ++i) q[i] = ldg_nc16(wp + (kb + 1) * 64 + 16 * i);
    }
    RDQ_STAGE_BEGIN(kb)
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      uint32_t h0, h1, h2, h3, h4, h5, h6, h7;
      cvt_e4m3x4(c[i].x, h0, h1);
      cvt_e4m3x4(c[i].y, h2, h3);
      cvt_e4m3x4(c[i].z, h4, h5);
      cvt_e4m3x4(c[i].w, h6, h7);
      st_chunk(row_base, sw, 4 * h + 2 * i, h0, h1, h2, h3);
      st_chunk(row_base, sw, 4 * h + 2 * i + 1, h4, h5, h6, h7);
    }
    RDQ_STAGE_END()
  }
}

// FP16 rows, rows beyond N (r < 0: zeros) and idle padding threads (j < 0: only the barrier protocol)
__device__ __forceinline__ void produce_fp16(GemmSmem &S, const GemmArgs &a, uint32_t b_base, int j, int h, int r, int nkb) {
  const uint32_t row_off = j >= 0 ? (j >> 3) * 1024 + (j & 7) * 128 : 0;
  const int sw = j & 7;
  const bool real = (j >= 0) && (r >= 0);
  const __half *wp = real ? a.w16 + 1ll * (r - a.n4 - a.n8) * a.K + h * 32 : nullptr;
  bool alive = true;
  uint4 q[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) q[i] = real ? ldg_nc16(wp + 8 * i) : make_uint4(0u, 0u, 0u, 0u);
  for (int kb = 0; kb < nkb; ++kb) {
    uint4 c[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) c[i] = q[i];
    if (real && kb + 1 < nkb) {
#pragma unroll
      for (int i = 0; i < 4; ++i) q[i] = ldg_nc16(wp + (kb + 1) * 64 + 8 * i);
    }
    RDQ_STAGE_BEGIN(kb)
    if (j >= 0) {
#pragma unroll
      for (int i = 0; i < 4; ++i) st_chunk(row_base, sw, 4 * h + i, c[i].x, c[i].y, c[i].z, c[i].w);
    }
    RDQ_STAGE_END()
  }
}

// MT = 128-token accumulators per CTA (1 or 2): with MT = 2 one dequantised weight stage
// feeds two MMAs groups, halving the conversion work per flop.
template <int MT>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_mixed_kernel(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ GemmArgs a) {
  constexpr int kStageAll = kStageA * MT;
  constexpr uint32_t kCols = kTmemCols * MT;
  extern __shared__ uint8_t smem_raw[];
  __shared__ GemmSmem S;
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t a_base = (raw_addr + 1023u) & ~1023u;  // swizzled tiles need 1024-byte alignment
  const uint32_t b_base = a_base + kStages * kStageAll;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int m0 = blockIdx.x * BM * MT;
  const int n0 = blockIdx.y * BN;
  const int N = a.n4 + a.n8 + a.n16;
  const int nkb = a.K / BK;

  if (tid == 0) {
    for (int i = 0; i < kStages; ++i) {
      mbar_init(smem_u32(&S.full[i]), kProducers + 1);
      mbar_init(smem_u32(&S.empty[i]), 1);
    }
    mbar_init(smem_u32(&S.accum), 1);
    S.abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&S.tmem_base)),
                 "r"(kCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (tid >= 64 && tid < 64 + BN) {
    const int j = tid - 64;
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
    // sort the tile rows by format (stable), one list per format
    int cnt[3] = {0, 0, 0};
    for (int round = 0; round < BN / 32; ++round) {
      const int j = round * 32 + lane;
      const int r = S.row_perm[j];
      const int f = (r >= 0 && r < a.n4) ? 0 : ((r >= a.n4 && r < a.n4 + a.n8) ? 1 : 2);
#pragma unroll
      for (int ff = 0; ff < 3; ++ff) {
        const uint32_t mask = __ballot_sync(0xffffffffu, f == ff);
        if (f == ff) S.order[ff][cnt[ff] + __popc(mask & ((1u << lane) - 1u))] = j;
        cnt[ff] += __popc(mask);
      }
    }
    if (lane == 0) {
      S.count[0] = cnt[0];
      S.count[1] = cnt[1];
      S.count[2] = cnt[2];
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = S.tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------- activation loads (TMA)
    if (lane == 0) {
      bool alive = true;
      for (int kb = 0; kb < nkb && alive; ++kb) {
        const int s = kb & (kStages - 1);
        if (kb >= kStages) alive = gemm_wait(&S.empty[s], ((kb / kStages) - 1) & 1, &S.abort_flag);
        if (!alive) break;
        const uint32_t full = smem_u32(&S.full[s]);
        mbar_arrive_expect_tx(full, kStageAll);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
          tma_load_2d(a_base + s * kStageAll + mt * kStageA, &xmap, kb * BK, m0 + mt * BM, full);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------------ MMA issue
    if (lane == 0) {
      constexpr uint32_t idesc = (1u << 4) | (static_cast<uint32_t>(BN >> 3) << 17) | (static_cast<uint32_t>(BM >> 4) << 24);
      bool alive = true;
      for (int kb = 0; kb < nkb && alive; ++kb) {
        const int s = kb & (kStages - 1);
        alive = gemm_wait(&S.full[s], (kb / kStages) & 1, &S.abort_flag);
        if (!alive) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint64_t db = make_desc_sw128(b_base + s * kStageB);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          const uint64_t da = make_desc_sw128(a_base + s * kStageAll + mt * kStageA);
#pragma unroll
          for (int k4 = 0; k4 < BK / 16; ++k4)
            umma_f16(tmem + mt * kTmemCols, da + 2 * k4, db + 2 * k4, idesc, (kb | k4) != 0 ? 1u : 0u);
        }
        umma_commit(smem_u32(&S.empty[s]));
      }
      umma_commit(smem_u32(&S.accum));
    }
  } else {
    // ------------------------------------------------------------- weight dequantisation
    // two threads per weight row (k halves); each format's rows are padded to whole warps
    const int pt = (tid - 64) >> 1, h = tid & 1;
    const int c0 = S.count[0], c1 = S.count[1], c2 = S.count[2];
    const int start1 = (c0 + 15) & ~15, start2 = start1 + ((c1 + 15) & ~15);
    if (pt < start1) {
      const int j = pt < c0 ? S.order[0][pt] : -1;
      if (j >= 0) produce_fp4(S, a, b_base, j, h, S.row_perm[j], nkb);
      else produce_fp16(S, a, b_base, -1, h, -1, nkb);
    } else if (pt < start2) {
      const int idx = pt - start1;
      const int j = idx < c1 ? S.order[1][idx] : -1;
      if (j >= 0) produce_fp8(S, a, b_base, j, h, S.row_perm[j], nkb);
      else produce_fp16(S, a, b_base, -1, h, -1, nkb);
    } else {
      const int idx = pt - start2;
      const int j = idx < c2 ? S.order[2][idx] : -1;
      produce_fp16(S, a, b_base, j, h, j >= 0 ? S.row_perm[j] : -1, nkb);
    }

    // ----------------------------------------------------------------------- epilogue
    if (warp >= 2 && warp < 6) {
      const bool ok = gemm_wait(&S.accum, 0, &S.abort_flag);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int q = warp & 3;  // tensor-memory lane quarter this warp may read
      if (ok) {
#pragma unroll 1
        for (int ci = 0; ci < MT * (BN / 32); ++ci) {
          const int mt = ci / (BN / 32), cc = ci % (BN / 32);
          const int m = m0 + mt * BM + q * 32 + lane;
          uint32_t r[32];
          tmem_ld32(tmem + (static_cast<uint32_t>(q * 32) << 16) + mt * kTmemCols + cc * 32, r);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          if (m < a.M) {
            __half *dst = a.y + 1ll * m * N + n0 + cc * 32;
            if (n0 + cc * 32 + 32 <= N && (N & 7) == 0) {
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
                *reinterpret_cast<uint4 *>(dst + v * 8) = make_uint4(o[0], o[1], o[2], o[3]);
              }
            } else {
              for (int e = 0; e < 32; ++e) {
                const int c = cc * 32 + e;
                if (n0 + c < N) dst[e] = __float2half_rn(fmaf(__uint_as_float(r[e]), S.colscale[c], S.colbias[c]));
              }
            }
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
  if (tid == 0 && S.abort_flag) atomicAdd(&g_gemm_aborts, 1);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

}  // namespace

int launch_gemm(const GemmArgs &a, cudaStream_t stream) {
  static EncodeTiledFn encode = nullptr;
  if (!encode) {
    cudaDriverEntryPointQueryResult qr;
    void *fn = nullptr;
    RDQ_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qr));
    RDQ_REQUIRE(fn != nullptr && qr == cudaDriverEntryPointSuccess, RDQ_E_CUDA, "cuTensorMapEncodeTiled is not available");
    encode = reinterpret_cast<EncodeTiledFn>(fn);
  }
  static bool attr_done[64] = {};
  int dev = 0;
  RDQ_CUDA(cudaGetDevice(&dev));
  const int smem1 = kStages * (kStageA + kStageB) + 1024;
  const int smem2 = kStages * (2 * kStageA + kStageB) + 1024;
  if (dev < 64 && !attr_done[dev]) {
    RDQ_CUDA(cudaFuncSetAttribute(gemm_mixed_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem1));
    RDQ_CUDA(cudaFuncSetAttribute(gemm_mixed_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem2));
    attr_done[dev] = true;
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
  // 256-token tiles once there are enough of them to fill the GPU
  const int ntile_n = (N + BN - 1) / BN;
  const bool two = ((a.M + 2 * BM - 1) / (2 * BM)) * ntile_n >= sm_count();
  if (two) {
    const dim3 grid((a.M + 2 * BM - 1) / (2 * BM), ntile_n);
    gemm_mixed_kernel<2><<<grid, kGemmThreads, smem2, stream>>>(xmap, a);
  } else {
    const dim3 grid((a.M + BM - 1) / BM, ntile_n);
    gemm_mixed_kernel<1><<<grid, kGemmThreads, smem1, stream>>>(xmap, a);
  }
  RDQ_CUDA(cudaGetLastError());
  return RDQ_OK;
}

}  // namespace rdq
