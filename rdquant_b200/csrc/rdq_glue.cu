// Decode-step glue between the mixed-precision linears of a transformer block: residual add +
// RMSNorm, per-head q/k RMSNorm + rotary embedding + KV-cache write, single-token attention over
// the cache, SiLU x mul.  The reference leaves these to the HuggingFace model code around its
// linear modules (rdquant/inference.py:689-708 is the module boundary; its end-to-end harness
// benchmarks/bench_e2e.py:103-155 captures that code in a CUDA graph); here they are small
// HBM/latency-bound kernels of their own because, at one token per step, each of the ~20 framework
// kernels between two linears costs more than the linear itself.
//
// Every kernel takes part in programmatic dependent launch the way the decode GEMV does: it lets
// its successor become resident at once (griddepcontrol.launch_dependents) -- so the next GEMV
// fills its weight rings while this kernel runs -- and reads its inputs only after
// griddepcontrol.wait.  All arithmetic is FP32 with one rounding to FP16 per stored value.
#include "rdq_kernels.cuh"

namespace rdq {

namespace {

__device__ __forceinline__ float block_sum(float v, float *smem) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();  // smem may still be read from a previous call
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  float t = (lane < nw) ? smem[lane] : 0.f;
  return warp_sum(t);
}

// ---- x (+= delta); out = rmsnorm(x) * w.  One CTA per row.
__global__ void __launch_bounds__(256) add_rmsnorm_kernel(__half *x, const __half *delta, const __half *w, __half *out,
                                                         int H, float eps) {
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  __half *xr = x + 1ll * blockIdx.x * H;
  const __half *dr = delta ? delta + 1ll * blockIdx.x * H : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) {
    uint4 v = reinterpret_cast<const uint4 *>(xr)[i];
    __half2 *h = reinterpret_cast<__half2 *>(&v);
    if (dr) {
      const uint4 d = reinterpret_cast<const uint4 *>(dr)[i];
      const __half2 *dh = reinterpret_cast<const __half2 *>(&d);
#pragma unroll
      for (int j = 0; j < 4; ++j) h[j] = __hadd2(h[j], dh[j]);
      reinterpret_cast<uint4 *>(xr)[i] = v;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __half22float2(h[j]);
      ss += f.x * f.x + f.y * f.y;
    }
  }
  ss = block_sum(ss, red);
  const float rs = rsqrtf(ss / H + eps);
  __half *orow = out + 1ll * blockIdx.x * H;
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) {
    const uint4 v = reinterpret_cast<const uint4 *>(xr)[i];
    const uint4 wv = reinterpret_cast<const uint4 *>(w)[i];
    const __half2 *h = reinterpret_cast<const __half2 *>(&v);
    const __half2 *wh = reinterpret_cast<const __half2 *>(&wv);
    uint4 o;
    __half2 *oh = reinterpret_cast<__half2 *>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __half22float2(h[j]);
      oh[j] = __hmul2(__floats2half2_rn(f.x * rs, f.y * rs), wh[j]);
    }
    reinterpret_cast<uint4 *>(orow)[i] = o;
  }
}

// ---- per head: (q, k) RMSNorm over head_dim (optional), rotary embedding, q -> q_out, k / v -> cache
// at position *pos.  grid = (nq + 2 nkv, B); one thread per rotary pair (i, i + dh / 2).
__global__ void __launch_bounds__(128) qk_rope_cache_kernel(const __half *qkv, const __half *qn, const __half *kn,
                                                           const __half *cos_t, const __half *sin_t, const long long *pos,
                                                           __half *q_out, __half *k_cache, __half *v_cache, int nq, int nkv,
                                                           int dh, int S, float eps) {
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  const int head = blockIdx.x, b = blockIdx.y, i = threadIdx.x, half = dh >> 1;
  const long long p = *pos;
  const __half *src = qkv + (1ll * b * (nq + 2 * nkv) + head) * dh;
  const float x0 = __half2float(src[i]), x1 = __half2float(src[i + half]);
  if (head >= nq + nkv) {  // v: copy
    __half *dst = v_cache + ((1ll * b * nkv + (head - nq - nkv)) * S + p) * dh;
    dst[i] = src[i];
    dst[i + half] = src[i + half];
    return;
  }
  const bool is_q = head < nq;
  const __half *nw = is_q ? qn : kn;
  float y0 = x0, y1 = x1;
  if (nw) {
    const float ss = block_sum(x0 * x0 + x1 * x1, red);
    const float rs = rsqrtf(ss / dh + eps);
    y0 = __half2float(__hmul(__float2half_rn(x0 * rs), nw[i]));
    y1 = __half2float(__hmul(__float2half_rn(x1 * rs), nw[i + half]));
  }
  const float c0 = __half2float(cos_t[p * dh + i]), s0 = __half2float(sin_t[p * dh + i]);
  const float c1 = __half2float(cos_t[p * dh + i + half]), s1 = __half2float(sin_t[p * dh + i + half]);
  const __half o0 = __float2half_rn(y0 * c0 - y1 * s0), o1 = __float2half_rn(y1 * c1 + y0 * s1);
  __half *dst = is_q ? q_out + (1ll * b * nq + head) * dh : k_cache + ((1ll * b * nkv + (head - nq)) * S + p) * dh;
  dst[i] = o0;
  dst[i + half] = o1;
}

// ---- attention of one new token over the cache, positions 0 .. *pos, split over blockIdx.x.
// grid = (nsplit, nkv, B); warp w serves the query heads kvh * group + w, w + 4, ... of its KV head;
// a lane owns dh / 32 consecutive dimensions.  Partial (max, sum, weighted values) per split go to
// scratch; attn_combine_kernel merges them.
constexpr int kAttnWarps = 4;
constexpr int kMaxDimsPerLane = 8;  // head_dim <= 256

__global__ void __launch_bounds__(kAttnWarps * 32) attn_split_kernel(const __half *q, const __half *k_cache,
                                                                    const __half *v_cache, const long long *pos,
                                                                    float *part, int nq, int nkv, int dh, int S, int chunk,
                                                                    float scale) {
  pdl_launch_dependents();
  pdl_wait();
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int nsplit = gridDim.x, group = nq / nkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int dpl = dh >> 5;  // dims per lane
  const int n = static_cast<int>(*pos) + 1;
  const int p0 = split * chunk, p1 = min(n, p0 + chunk);
  const __half *kb = k_cache + (1ll * b * nkv + kvh) * S * dh + lane * dpl;
  const __half *vb = v_cache + (1ll * b * nkv + kvh) * S * dh + lane * dpl;
  for (int hq = warp; hq < group; hq += kAttnWarps) {
    const int head = kvh * group + hq;
    float qv[kMaxDimsPerLane], acc[kMaxDimsPerLane];
    const __half *qp = q + (1ll * b * nq + head) * dh + lane * dpl;
#pragma unroll
    for (int j = 0; j < kMaxDimsPerLane; ++j) {
      qv[j] = j < dpl ? __half2float(qp[j]) * scale : 0.f;
      acc[j] = 0.f;
    }
    float m = -INFINITY, l = 0.f;
    for (int p = p0; p < p1; ++p) {
      float kf[kMaxDimsPerLane], vf[kMaxDimsPerLane];
      if (dpl == 4) {  // head_dim 128: one 8-byte load per lane and tensor
        const uint2 kr = *reinterpret_cast<const uint2 *>(kb + 1ll * p * dh);
        const uint2 vr = *reinterpret_cast<const uint2 *>(vb + 1ll * p * dh);
        const float2 k01 = __half22float2(*reinterpret_cast<const __half2 *>(&kr.x));
        const float2 k23 = __half22float2(*reinterpret_cast<const __half2 *>(&kr.y));
        const float2 v01 = __half22float2(*reinterpret_cast<const __half2 *>(&vr.x));
        const float2 v23 = __half22float2(*reinterpret_cast<const __half2 *>(&vr.y));
        kf[0] = k01.x; kf[1] = k01.y; kf[2] = k23.x; kf[3] = k23.y;
        vf[0] = v01.x; vf[1] = v01.y; vf[2] = v23.x; vf[3] = v23.y;
      } else {
#pragma unroll
        for (int j = 0; j < kMaxDimsPerLane; ++j) {
          kf[j] = j < dpl ? __half2float(kb[1ll * p * dh + j]) : 0.f;
          vf[j] = j < dpl ? __half2float(vb[1ll * p * dh + j]) : 0.f;
        }
      }
      float s = 0.f;
#pragma unroll
      for (int j = 0; j < kMaxDimsPerLane; ++j)
        if (j < dpl) s += qv[j] * kf[j];
      s = warp_sum(s);
      const float mn = fmaxf(m, s);
      const float corr = __expf(m - mn), w = __expf(s - mn);
      l = l * corr + w;
#pragma unroll
      for (int j = 0; j < kMaxDimsPerLane; ++j)
        if (j < dpl) acc[j] = acc[j] * corr + w * vf[j];
      m = mn;
    }
    float *dst = part + ((1ll * b * nq + head) * nsplit + split) * (dh + 2);
    if (lane == 0) {
      dst[0] = m;
      dst[1] = l;
    }
#pragma unroll
    for (int j = 0; j < kMaxDimsPerLane; ++j)
      if (j < dpl) dst[2 + lane * dpl + j] = acc[j];
  }
}

// grid = (nq, B), one thread per dimension
__global__ void __launch_bounds__(256) attn_combine_kernel(const float *part, __half *out, int nq, int dh, int nsplit) {
  pdl_launch_dependents();
  pdl_wait();
  const int head = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
  const float *src = part + (1ll * b * nq + head) * nsplit * (dh + 2);
  float m = -INFINITY;
  for (int s = 0; s < nsplit; ++s) m = fmaxf(m, src[s * (dh + 2)]);
  float l = 0.f, a = 0.f;
  for (int s = 0; s < nsplit; ++s) {
    const float ms = src[s * (dh + 2)];
    if (ms == -INFINITY) continue;
    const float w = __expf(ms - m);
    l += src[s * (dh + 2) + 1] * w;
    a += src[s * (dh + 2) + 2 + d] * w;
  }
  out[(1ll * b * nq + head) * dh + d] = __float2half_rn(a / l);
}

// ---- out[b, f] = silu(gu[b, f]) * gu[b, F + f]
__global__ void __launch_bounds__(256) silu_mul_kernel(const __half *gu, __half *out, int B, int F) {
  pdl_launch_dependents();
  pdl_wait();
  const long long total = 1ll * B * (F / 8);
  for (long long i = 1ll * blockIdx.x * blockDim.x + threadIdx.x; i < total; i += 1ll * gridDim.x * blockDim.x) {
    const int b = static_cast<int>(i / (F / 8)), j = static_cast<int>(i - 1ll * b * (F / 8));
    const uint4 g = reinterpret_cast<const uint4 *>(gu + 2ll * b * F)[j];
    const uint4 u = reinterpret_cast<const uint4 *>(gu + 2ll * b * F + F)[j];
    const __half2 *gh = reinterpret_cast<const __half2 *>(&g);
    const __half2 *uh = reinterpret_cast<const __half2 *>(&u);
    uint4 o;
    __half2 *oh = reinterpret_cast<__half2 *>(&o);
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const float2 a = __half22float2(gh[t]), c = __half22float2(uh[t]);
      // silu in FP32, rounded to FP16 before the product like the framework's two kernels
      const __half2 s = __floats2half2_rn(a.x / (1.f + __expf(-a.x)), a.y / (1.f + __expf(-a.y)));
      oh[t] = __hmul2(s, __floats2half2_rn(c.x, c.y));
    }
    reinterpret_cast<uint4 *>(out + 1ll * b * F)[j] = o;
  }
}

template <typename... Args>
int launch_pdl(void (*kernel)(Args...), dim3 grid, dim3 block, bool pdl, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  RDQ_CUDA(cudaLaunchKernelEx(&cfg, kernel, args...));
  return RDQ_OK;
}

}  // namespace

int launch_add_rmsnorm(__half *x, const __half *delta, const __half *w, __half *out, int B, int H, float eps, bool pdl,
                       cudaStream_t stream) {
  return launch_pdl(add_rmsnorm_kernel, dim3(B), dim3(256), pdl, stream, x, delta, w, out, H, eps);
}

int launch_qk_rope_cache(const __half *qkv, const __half *qn, const __half *kn, const __half *cos_t, const __half *sin_t,
                         const long long *pos, __half *q_out, __half *k_cache, __half *v_cache, int B, int nq, int nkv,
                         int dh, int S, float eps, bool pdl, cudaStream_t stream) {
  return launch_pdl(qk_rope_cache_kernel, dim3(nq + 2 * nkv, B), dim3(dh / 2), pdl, stream, qkv, qn, kn, cos_t, sin_t, pos,
                    q_out, k_cache, v_cache, nq, nkv, dh, S, eps);
}

int attn_chunk() { return 32; }

int launch_attn_decode(const __half *q, const __half *k_cache, const __half *v_cache, const long long *pos, float *scratch,
                       __half *out, int B, int nq, int nkv, int dh, int S, float scale, bool pdl, cudaStream_t stream) {
  const int chunk = attn_chunk();
  const int nsplit = (S + chunk - 1) / chunk;
  int rc = launch_pdl(attn_split_kernel, dim3(nsplit, nkv, B), dim3(kAttnWarps * 32), pdl, stream, q, k_cache, v_cache, pos,
                      scratch, nq, nkv, dh, S, chunk, scale);
  if (rc != RDQ_OK) return rc;
  return launch_pdl(attn_combine_kernel, dim3(nq, B), dim3(dh), pdl, stream, static_cast<const float *>(scratch), out, nq, dh,
                    nsplit);
}

int launch_silu_mul(const __half *gu, __half *out, int B, int F, bool pdl, cudaStream_t stream) {
  const long long total = 1ll * B * (F / 8);
  const int blocks = static_cast<int>(std::min<long long>((total + 255) / 256, 4ll * sm_count()));
  return launch_pdl(silu_mul_kernel, dim3(blocks), dim3(256), pdl, stream, gu, out, B, F);
}

}  // namespace rdq
