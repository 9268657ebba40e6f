// Encoders: a float weight group [n, K] -> the packed checkpoint tensors of the NVFP4 or FP8
// format, bit for bit what the reference's CPU encoders produce
// (rdquant/core/formats.py:84-142 nvfp4_quantize, :166-193 fp8_quantize; byte layout
// rdquant/integrations/hf_export.py:81-102), plus the per-row sum of squared reconstruction
// errors that the per-channel MSE of the format search needs
// (rdquant/core/formats.py:414-436 compute_mse_2d: mean over the row of (w - dequant)^2).
//
// One warp per row, a lane per block of 16 consecutive k (K % 16 == 0, so the reference's
// blocks over the flattened group coincide with blocks inside rows).  Arithmetic follows
// the reference operation by operation in IEEE float32: block scale =
// e4m3(clamp(absmax / 6)), ratio = v / scale (scale 0 -> 1), code = number of grid midpoints
// strictly below |ratio| (ties go to the smaller magnitude) + 8 if ratio < 0; FP8 scale =
// absmax(group) / 448 (0 -> 1), byte = e4m3(clamp(v / scale)).  The E4M3 rounding is the
// hardware converter's round-to-nearest-even, the same as torch.float8_e4m3fn's.
//
// HBM-bound elementwise work: reads 4 (f32) or 2 (f16) bytes per element, writes 0.56 / 1.
#include <cuda_fp8.h>

#include "rdq_kernels.cuh"

namespace rdq {

namespace {

__device__ __forceinline__ float load_elem(const float *p, long long i) { return p[i]; }
__device__ __forceinline__ float load_elem(const __half *p, long long i) { return __half2float(p[i]); }
// 16 consecutive elements starting at a multiple of 16 (the tensor is 16-byte aligned)
__device__ __forceinline__ void load16(const float *p, long long i, float (&v)[16]) {
  const float4 *q = reinterpret_cast<const float4 *>(p + i);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float4 t = __ldg(q + j);
    v[4 * j] = t.x; v[4 * j + 1] = t.y; v[4 * j + 2] = t.z; v[4 * j + 3] = t.w;
  }
}
__device__ __forceinline__ void load16(const __half *p, long long i, float (&v)[16]) {
  const uint4 *q = reinterpret_cast<const uint4 *>(p + i);
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const uint4 t = __ldg(q + j);
    const uint32_t u[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&u[e]));
      v[8 * j + 2 * e] = f.x;
      v[8 * j + 2 * e + 1] = f.y;
    }
  }
}

__device__ __forceinline__ uint8_t to_e4m3(float v) {
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
}
__device__ __forceinline__ float from_e4m3(uint8_t b) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(b), __NV_E4M3);
  return __half2float(__half(h));
}
__device__ __forceinline__ float clamp448(float v) { return fminf(fmaxf(v, -448.f), 448.f); }

// deterministic max of non-negative floats through their bit patterns
__device__ __forceinline__ void atomic_max_nonneg(float *addr, float v) {
  atomicMax(reinterpret_cast<unsigned int *>(addr), __float_as_uint(v));
}

template <typename T>
__global__ void __launch_bounds__(256) quantize_nvfp4_kernel(const T *__restrict__ w, int n, int K, uint8_t *__restrict__ codes,
                                                             uint8_t *__restrict__ scales, float *__restrict__ row_sqerr,
                                                             float *__restrict__ max_scale) {
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int nblk = K >> 4;
  float top = 0.f;
  for (int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; row < n; row += warps) {
    float err = 0.f;
    for (int b = lane; b < nblk; b += 32) {
      const long long base = 1ll * row * K + 16 * b;
      float v[16];
      load16(w, base, v);
      float amax = 0.f;
#pragma unroll
      for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
      const uint8_t sbits = to_e4m3(clamp448(__fdiv_rn(amax, 6.f)));
      const float scale = from_e4m3(sbits);
      const float divisor = (scale == 0.f) ? 1.f : scale;
      top = fmaxf(top, scale);
      uint32_t packed[2] = {0u, 0u};
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float ratio = __fdiv_rn(v[i], divisor);
        const float mag = fabsf(ratio);
        const int m = (mag > 0.25f) + (mag > 0.75f) + (mag > 1.25f) + (mag > 1.75f) + (mag > 2.5f) + (mag > 3.5f) + (mag > 5.0f);
        const int code = m + ((ratio < 0.f) ? 8 : 0);
        packed[i >> 3] |= static_cast<uint32_t>(code) << (4 * (i & 7));
        // grid value: 0, .5, 1, 1.5 (m / 2) then 2, 3, 4, 6
        const float g = (m < 4) ? 0.5f * m : (m == 7 ? 6.f : static_cast<float>(m - 2));
        const float rec = __fmul_rn((ratio < 0.f) ? -g : g, scale);
        const float d = v[i] - rec;
        err = fmaf(d, d, err);
      }
      *reinterpret_cast<uint2 *>(codes + 1ll * row * (K >> 1) + 8 * b) = make_uint2(packed[0], packed[1]);
      scales[1ll * row * nblk + b] = sbits;
    }
    if (row_sqerr) {
      err = warp_sum(err);
      if (lane == 0) row_sqerr[row] = err;
    }
  }
  if (max_scale) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, o));
    if (lane == 0 && top > 0.f) atomic_max_nonneg(max_scale, top);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) absmax_kernel(const T *__restrict__ w, long long count, float *__restrict__ out) {
  float m = 0.f;
  for (long long i = 1ll * blockIdx.x * blockDim.x + threadIdx.x; i < count; i += 1ll * gridDim.x * blockDim.x)
    m = fmaxf(m, fabsf(load_elem(w, i)));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0 && m > 0.f) atomic_max_nonneg(out, m);
}

template <typename T>
__global__ void __launch_bounds__(256) quantize_fp8_kernel(const T *__restrict__ w, int n, int K, const float *__restrict__ absmax,
                                                           uint8_t *__restrict__ out, float *__restrict__ scale_out,
                                                           float *__restrict__ row_sqerr) {
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  float scale = __fdiv_rn(*absmax, 448.f);
  if (scale == 0.f) scale = 1.f;
  for (int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; row < n; row += warps) {
    float err = 0.f;
    for (int b = lane; b < (K >> 4); b += 32) {
      const long long base = 1ll * row * K + 16 * b;
      uint32_t o[4] = {0u, 0u, 0u, 0u};
      float v[16];
      load16(w, base, v);
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const uint8_t q = to_e4m3(clamp448(__fdiv_rn(v[i], scale)));
        o[i >> 2] |= static_cast<uint32_t>(q) << (8 * (i & 3));
        const float d = v[i] - __fmul_rn(from_e4m3(q), scale);
        err = fmaf(d, d, err);
      }
      *reinterpret_cast<uint4 *>(out + base) = make_uint4(o[0], o[1], o[2], o[3]);
    }
    if (lane == 0 && scale_out) scale_out[row] = scale;
    if (row_sqerr) {
      err = warp_sum(err);
      if (lane == 0) row_sqerr[row] = err;
    }
  }
}

int grid_for_rows(int n) {
  const long long want = (1ll * n + 7) / 8;  // 8 warps per block
  const long long cap = 1ll * sm_count() * 8;
  return static_cast<int>(want < cap ? (want > 0 ? want : 1) : cap);
}

}  // namespace

int launch_quantize_nvfp4(const void *w, bool w_is_f32, int n, int K, uint8_t *codes, uint8_t *scales, float *row_sqerr,
                          float *max_scale, cudaStream_t stream) {
  if (max_scale) RDQ_CUDA(cudaMemsetAsync(max_scale, 0, sizeof(float), stream));
  const int grid = grid_for_rows(n);
  if (w_is_f32)
    quantize_nvfp4_kernel<float><<<grid, 256, 0, stream>>>(static_cast<const float *>(w), n, K, codes, scales, row_sqerr, max_scale);
  else
    quantize_nvfp4_kernel<__half><<<grid, 256, 0, stream>>>(static_cast<const __half *>(w), n, K, codes, scales, row_sqerr,
                                                           max_scale);
  RDQ_CUDA(cudaGetLastError());
  return RDQ_OK;
}

int launch_quantize_fp8(const void *w, bool w_is_f32, int n, int K, uint8_t *out, float *scale_out, float *row_sqerr,
                        float *absmax_scratch, cudaStream_t stream) {
  RDQ_CUDA(cudaMemsetAsync(absmax_scratch, 0, sizeof(float), stream));
  const long long count = 1ll * n * K;
  long long blocks = (count + 256 * 16 - 1) / (256 * 16);
  const long long cap = 1ll * sm_count() * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  const int grid = grid_for_rows(n);
  if (w_is_f32) {
    absmax_kernel<float><<<static_cast<int>(blocks), 256, 0, stream>>>(static_cast<const float *>(w), count, absmax_scratch);
    quantize_fp8_kernel<float><<<grid, 256, 0, stream>>>(static_cast<const float *>(w), n, K, absmax_scratch, out, scale_out,
                                                        row_sqerr);
  } else {
    absmax_kernel<__half><<<static_cast<int>(blocks), 256, 0, stream>>>(static_cast<const __half *>(w), count, absmax_scratch);
    quantize_fp8_kernel<__half><<<grid, 256, 0, stream>>>(static_cast<const __half *>(w), n, K, absmax_scratch, out, scale_out,
                                                         row_sqerr);
  }
  RDQ_CUDA(cudaGetLastError());
  return RDQ_OK;
}

}  // namespace rdq
