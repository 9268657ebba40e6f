// Any-shape decode GEMV (M <= 16): one warp per permuted weight row, direct
// global loads, FP32 accumulation, warp-shuffle reduction, scatter store to
// y[m, perm[row]].  This is the fallback for shapes the TMA-staged stream
// kernel does not take (groups that are not multiples of 16 rows, K not a
// multiple of 256, unaligned pointers); same arithmetic contract.
//
// Reference behaviour replaced: rdquant/ops.py:55-66 (per-group dequant +
// F.linear + cat + index_select) and kernel K1 rdquant/csrc/fused_gemv.cu:1198-1242.
#include "rdq_kernels.cuh"

namespace rdq {

namespace {

template <int MP>
__device__ __forceinline__ void fma16(float (&acc)[MP], const float (&w)[16], const __half *x,
                                      int M, int K, int k0) {
#pragma unroll
  for (int m = 0; m < MP; ++m) {
    if (m < M) {
      const uint4 *xp = reinterpret_cast<const uint4 *>(x + 1ll * m * K + k0);
      const uint4 xa = __ldg(xp), xb = __ldg(xp + 1);
      const uint32_t xs[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
      float s = acc[m];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float2 f = h2_to_f2(xs[i]);
        s = fmaf(w[2 * i], f.x, s);
        s = fmaf(w[2 * i + 1], f.y, s);
      }
      acc[m] = s;
    }
  }
}

template <int MP>
__global__ void __launch_bounds__(256) gemv_generic_kernel(GemvArgs a) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int N = a.n4 + a.n8 + a.n16;
  if (row >= N) return;
  const int K = a.K, M = a.M;
  float acc[MP];
#pragma unroll
  for (int m = 0; m < MP; ++m) acc[m] = 0.f;
  float out_scale = 1.f;

  if (row < a.n4) {
    const uint8_t *wrow = a.w4 + 1ll * row * (K >> 1);
    const uint8_t *srow = a.s4 + 1ll * row * (K >> 4);
    for (int b = lane; b < (K >> 4); b += 32) {
      const uint2 q = __ldg(reinterpret_cast<const uint2 *>(wrow + b * 8));
      const float sc = e4m3_to_float(srow[b]) * a.global4;
      uint32_t h[8];
      cvt_e2m1x8(q.x, h[0], h[1], h[2], h[3]);
      cvt_e2m1x8(q.y, h[4], h[5], h[6], h[7]);
      float w[16];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float2 f = h2_to_f2(h[i]);
        // the oracle's weight is f16(LUT * scale); round so both paths multiply the same value
        w[2 * i] = __half2float(__float2half_rn(f.x * sc));
        w[2 * i + 1] = __half2float(__float2half_rn(f.y * sc));
      }
      fma16<MP>(acc, w, a.x, M, K, b << 4);
    }
  } else if (row < a.n4 + a.n8) {
    const int rr = row - a.n4;
    const uint8_t *wrow = a.w8 + 1ll * rr * K;
    out_scale = a.s8[rr];
    if ((K & 15) == 0) {
      for (int c = lane; c < (K >> 4); c += 32) {
        const uint4 q = __ldg(reinterpret_cast<const uint4 *>(wrow + c * 16));
        const uint32_t ws[4] = {q.x, q.y, q.z, q.w};
        float w[16];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint32_t h01, h23;
          cvt_e4m3x4(ws[i], h01, h23);
          const float2 f0 = h2_to_f2(h01), f1 = h2_to_f2(h23);
          w[4 * i] = f0.x;
          w[4 * i + 1] = f0.y;
          w[4 * i + 2] = f1.x;
          w[4 * i + 3] = f1.y;
        }
        fma16<MP>(acc, w, a.x, M, K, c << 4);
      }
    } else {
      for (int k = lane; k < K; k += 32) {
        const float w = e4m3_to_float(wrow[k]);
#pragma unroll
        for (int m = 0; m < MP; ++m)
          if (m < M) acc[m] = fmaf(w, __half2float(a.x[1ll * m * K + k]), acc[m]);
      }
    }
  } else {
    const int rr = row - a.n4 - a.n8;
    const __half *wrow = a.w16 + 1ll * rr * K;
    if ((K & 15) == 0) {
      for (int c = lane; c < (K >> 4); c += 32) {
        const uint4 *wp = reinterpret_cast<const uint4 *>(wrow + c * 16);
        const uint4 qa = __ldg(wp), qb = __ldg(wp + 1);
        const uint32_t ws[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
        float w[16];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float2 f = h2_to_f2(ws[i]);
          w[2 * i] = f.x;
          w[2 * i + 1] = f.y;
        }
        fma16<MP>(acc, w, a.x, M, K, c << 4);
      }
    } else {
      for (int k = lane; k < K; k += 32) {
        const float w = __half2float(wrow[k]);
#pragma unroll
        for (int m = 0; m < MP; ++m)
          if (m < M) acc[m] = fmaf(w, __half2float(a.x[1ll * m * K + k]), acc[m]);
      }
    }
  }

  const int col = a.perm ? a.perm[row] : row;
  const float b = a.bias ? __half2float(a.bias[col]) : 0.f;
#pragma unroll
  for (int m = 0; m < MP; ++m) {
    const float s = warp_sum(acc[m]);
    if (m < M && lane == 0) a.y[1ll * m * N + col] = __float2half_rn(fmaf(s, out_scale, b));
  }
}

}  // namespace

int launch_gemv_generic(const GemvArgs &a, cudaStream_t stream) {
  const int N = a.n4 + a.n8 + a.n16;
  if (N == 0 || a.M == 0) return RDQ_OK;
  const unsigned blocks = static_cast<unsigned>((N + 7) / 8);
  if (a.M <= 1) gemv_generic_kernel<1><<<blocks, 256, 0, stream>>>(a);
  else if (a.M <= 2) gemv_generic_kernel<2><<<blocks, 256, 0, stream>>>(a);
  else if (a.M <= 4) gemv_generic_kernel<4><<<blocks, 256, 0, stream>>>(a);
  else if (a.M <= 8) gemv_generic_kernel<8><<<blocks, 256, 0, stream>>>(a);
  else gemv_generic_kernel<16><<<blocks, 256, 0, stream>>>(a);
  RDQ_CUDA(cudaGetLastError());
  return RDQ_OK;
}

}  // namespace rdq
