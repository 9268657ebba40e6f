// Bit-exact dequantisation of a packed mixed-precision layer to FP16 [N, K] in
// original channel order.  HBM-bound elementwise kernel: reads the packed
// bytes once, writes 2*N*K bytes once; each thread owns one 16-element run
// (one NVFP4 scale block) of one output row.
//
// Arithmetic follows the reference oracle exactly:
//   NVFP4  f16( f32(LUT[code]) * f32(e4m3 scale) )        rdquant/core/formats.py:145-159
//   FP8    f16( f32(e4m3 byte) * scale[channel] )          rdquant/inference.py:104-109
//   FP16   bf16 -> f32 -> f16 (or a plain copy of f16)     rdquant/inference.py:111-113
// and the row gather is QuantizedWeight.dequantize's cat()[inv_perm]
// (rdquant/quantize.py:56-69).
#include "rdq_kernels.cuh"

namespace rdq {

namespace {

struct DequantArgs {
  const uint8_t *w4;
  const uint8_t *s4;
  float global4;
  const uint8_t *w8;
  const float *s8;
  const void *w16;
  int w16_is_bf16;
  const int32_t *inv_perm;
  void *out;
  int out_is_f32;
  int n4, n8, n16, K;
};

// `vec` says the row pitch keeps every 16-element run 32 / 64-byte aligned (K % 16 == 0);
// otherwise the run is stored element by element, full runs included.
__device__ __forceinline__ void store16(__half *dst, const float (&v)[16], int valid, bool vec) {
  if (vec) {
    __half2 o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
    uint4 *d4 = reinterpret_cast<uint4 *>(dst);
    d4[0] = *reinterpret_cast<uint4 *>(&o[0]);
    d4[1] = *reinterpret_cast<uint4 *>(&o[4]);
  } else {
    for (int i = 0; i < valid; ++i) dst[i] = __float2half_rn(v[i]);
  }
}
__device__ __forceinline__ void store16(float *dst, const float (&v)[16], int valid, bool vec) {
  if (vec) {
    float4 *d4 = reinterpret_cast<float4 *>(dst);
#pragma unroll
    for (int i = 0; i < 4; ++i) d4[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
  } else {
    for (int i = 0; i < valid; ++i) dst[i] = v[i];
  }
}

// OutT = __half: the operator's weight (products rounded to f16, round to nearest even).
// OutT = float : the unrounded FP32 product, what formats.dequantize returns.
template <typename OutT>
__global__ void __launch_bounds__(256) dequant_kernel(DequantArgs a) {
  const int K = a.K;
  const int chunks = (K + 15) >> 4;
  const bool vec = (K & 15) == 0;
  const long long total = 1ll * (a.n4 + a.n8 + a.n16) * chunks;
  OutT *out = reinterpret_cast<OutT *>(a.out);
  for (long long item = 1ll * blockIdx.x * blockDim.x + threadIdx.x; item < total;
       item += 1ll * gridDim.x * blockDim.x) {
    const int n = static_cast<int>(item / chunks);
    const int c = static_cast<int>(item - 1ll * n * chunks);
    const int r = a.inv_perm ? a.inv_perm[n] : n;
    const int k0 = c << 4;
    const int valid = min(16, K - k0);
    float v[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = 0.f;
    if (r < a.n4) {
      // K % 16 == 0 is a precondition of the NVFP4 layout.
      const uint8_t *src = a.w4 + 1ll * r * (K >> 1) + (k0 >> 1);
      const float sc = e4m3_to_float(a.s4[1ll * r * (K >> 4) + c]) * a.global4;
      const uint2 q = *reinterpret_cast<const uint2 *>(src);
      uint32_t h[8];
      cvt_e2m1x8(q.x, h[0], h[1], h[2], h[3]);
      cvt_e2m1x8(q.y, h[4], h[5], h[6], h[7]);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float2 f = h2_to_f2(h[i]);
        v[2 * i] = f.x * sc;
        v[2 * i + 1] = f.y * sc;
      }
    } else if (r < a.n4 + a.n8) {
      const int rr = r - a.n4;
      const float sc = a.s8[rr];
      const uint8_t *src = a.w8 + 1ll * rr * K + k0;
      if (vec) {
        const uint4 q = *reinterpret_cast<const uint4 *>(src);
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint32_t h01, h23;
          cvt_e4m3x4(w[i], h01, h23);
          const float2 f0 = h2_to_f2(h01), f1 = h2_to_f2(h23);
          v[4 * i] = f0.x * sc;
          v[4 * i + 1] = f0.y * sc;
          v[4 * i + 2] = f1.x * sc;
          v[4 * i + 3] = f1.y * sc;
        }
      } else {
        for (int i = 0; i < valid; ++i) v[i] = e4m3_to_float(src[i]) * sc;
      }
    } else {
      const int rr = r - a.n4 - a.n8;
      if (a.w16_is_bf16) {
        const __nv_bfloat16 *src = reinterpret_cast<const __nv_bfloat16 *>(a.w16) + 1ll * rr * K + k0;
        for (int i = 0; i < valid; ++i) v[i] = __half2float(__float2half_rn(__bfloat162float(src[i])));
      } else {
        const __half *src = reinterpret_cast<const __half *>(a.w16) + 1ll * rr * K + k0;
        for (int i = 0; i < valid; ++i) v[i] = __half2float(src[i]);
      }
    }
    store16(out + 1ll * n * K + k0, v, valid, vec);
  }
}

}  // namespace

int launch_dequant(const void *w_fp4, const void *w_fp4_scales, float global4, const void *w_fp8,
                   const float *w_fp8_scales, const void *w_fp16, int fp16_is_bf16,
                   const int32_t *inv_perm, void *w_out, int out_is_f32, int n4, int n8, int n16,
                   int K, cudaStream_t stream) {
  DequantArgs a;
  a.w4 = static_cast<const uint8_t *>(w_fp4);
  a.s4 = static_cast<const uint8_t *>(w_fp4_scales);
  a.global4 = global4;
  a.w8 = static_cast<const uint8_t *>(w_fp8);
  a.s8 = w_fp8_scales;
  a.w16 = w_fp16;
  a.w16_is_bf16 = fp16_is_bf16;
  a.inv_perm = inv_perm;
  a.out = w_out;
  a.out_is_f32 = out_is_f32;
  a.n4 = n4;
  a.n8 = n8;
  a.n16 = n16;
  a.K = K;
  const long long total = 1ll * (n4 + n8 + n16) * ((K + 15) / 16);
  if (total == 0) return RDQ_OK;
  long long blocks = (total + 255) / 256;
  const long long cap = 1ll * sm_count() * 32;
  if (blocks > cap) blocks = cap;
  if (out_is_f32) {
    dequant_kernel<float><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(a);
  } else {
    dequant_kernel<__half><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(a);
  }
  RDQ_CUDA(cudaGetLastError());
  return RDQ_OK;
}

}  // namespace rdq
