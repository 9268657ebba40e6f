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

#include <utility>
#include <vector>

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
                                                         int B, int H, float eps) {
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  if (static_cast<int>(blockIdx.x) >= B) {  // the grid has a CTA per SM (see linger())
    linger(1500);
    return;
  }
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
  // every CTA takes an equal, contiguous share of the 16-byte vectors, so that (nearly) all SMs
  // work and leave together
  const long long total = 1ll * B * (F / 8);
  const long long per = (total + gridDim.x - 1) / gridDim.x;
  const long long lo = per * blockIdx.x, hi = lo + per < total ? lo + per : total;
  if (lo >= total) {  // the grid has a CTA per SM (see linger())
    linger(1500);
    return;
  }
  for (long long i = lo + threadIdx.x; i < hi; i += blockDim.x) {
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

// ---- q/k RMSNorm + rotary embedding + KV-cache write + attention of the new token over the
// cache + merge of the splits, in one launch.
// One CTA per SM, 128 threads: CTA c is (sequence, KV head) c / nsplit and split c % nsplit, with
// nsplit = SMs / (sequences x KV heads) (at most 16); it serves the `group` query heads of its KV
// head over the cache rows [split * chunk, (split + 1) * chunk) with chunk = the n = *pos + 1
// rows divided by nsplit, rounded up to 32; warp w takes the heads w, w + 4, ...
//   1. every CTA normalises and rotates its query heads into shared memory (FP16-rounded like the
//      stored q of the separate kernel, times `scale`); the CTA whose rows include *pos does the
//      same for the new key, copies the new value, and writes both to the cache and to its tile.
//   2. K and V rows go to shared memory in tiles of TP rows by cp.async, two tiles in flight, so a
//      CTA pays one memory round trip, not one per row.
//   3. scores with one lane per row (K rows padded by 16 bytes against bank conflicts), online
//      softmax per 32 rows, then P x V with one lane per DH / 32 dimensions.
//   4. partial (max, sum, values) per split go to scratch; the last CTA of a (b, kvh) to arrive
//      (counter in scratch, left at zero again) merges them and writes out [B, nq * dh].
constexpr int kFusedAttnThreads = 256;
constexpr int kFusedAttnWarps = kFusedAttnThreads / 32;
constexpr int kFusedAttnMaxSplit = 16;  // one batch of merge loads at head_dim <= 128

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

template <int DH>
__global__ void __launch_bounds__(kFusedAttnThreads, 2) rope_attn_kernel(
    const __half *qkv, const __half *qn, const __half *kn, const __half *cos_t, const __half *sin_t, const long long *pos,
    __half *k_cache, __half *v_cache, float *part, int *counters, __half *out, int nq, int nkv, int S, float scale,
    float eps, int nsplit, int npair) {
  constexpr int TP = 8192 / DH;        // rows per tile: 16 KB of V, a little more of K
  constexpr int KP = 2 * DH + 16;      // K row pitch in shared memory (bytes)
  constexpr int VP = 2 * DH;
  constexpr int HALF = DH / 2;
  constexpr int DPL = DH / 32;         // dimensions per lane in P x V
  constexpr int VPR = DH / 8;          // 16-byte vectors per row
  extern __shared__ __align__(16) uint8_t smem[];
  uint8_t *ks = smem;                           // [2][TP][KP]
  uint8_t *vs = smem + 2 * TP * KP;             // [2][TP][VP]
  float *qs = reinterpret_cast<float *>(vs + 2 * TP * VP);  // [group][DH]
  constexpr int W = kFusedAttnWarps;
  constexpr int PR = DH + 4;  // a partial: max, sum, two unused, then the DH weighted values (16-byte aligned)
  __shared__ int s_last;

  pdl_launch_dependents();
  pdl_wait();
  // CTA -> (sequence, KV head, split).  The grid has one CTA per SM (or one per (sequence, KV
  // head) when those outnumber the SMs); CTAs beyond the work linger (see below).
  const int pair = static_cast<int>(blockIdx.x) / nsplit, split = static_cast<int>(blockIdx.x) - pair * nsplit;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (pair >= npair) {
    linger(4000);
    return;
  }
  const int kvh = pair % nkv, b = pair / nkv;
  const int group = nq / nkv;
  // Warp -> (query head, slice of the rows): hp heads are served at a time, by nsl warps each;
  // the warps of a head take every nsl-th block of 32 rows and are merged in shared memory.
  const int hp = min(group, W), nsl = max(1, W / hp);
  const int slice = warp / hp, head0 = warp - slice * hp;
  const bool active = slice < nsl;
  float *mrg = qs + group * DH;  // [W][2][PR]: partials of the slices above 0
  // Loads that do not depend on the position go first, so that they share a round trip with it:
  // the raw values of this warp's first query head and the norm weights.
  const __half *row = qkv + 1ll * b * (nq + 2 * nkv) * DH;
  float qx0[HALF / 32], qx1[HALF / 32], qw0[HALF / 32], qw1[HALF / 32];
  auto load_row = [&](const __half *src, float (&x0)[HALF / 32], float (&x1)[HALF / 32]) {
#pragma unroll
    for (int t = 0; t < HALF / 32; ++t) {
      x0[t] = __half2float(src[lane + 32 * t]);
      x1[t] = __half2float(src[lane + 32 * t + HALF]);
    }
  };
  if (slice == 0) load_row(row + 1ll * (kvh * group + head0) * DH, qx0, qx1);
  if (qn) load_row(qn, qw0, qw1);
  const long long p_new = *pos;
  const int n = static_cast<int>(p_new) + 1;
  const int chunk = (n + nsplit - 1) / nsplit;
  const int used = (n + chunk - 1) / chunk;
  if (split >= used) {
    linger(4000);
    return;
  }
  const int p0 = split * chunk, p1 = min(n, p0 + chunk);
  const int ntile = (p1 - p0 + TP - 1) / TP;
  const __half *kb = k_cache + (1ll * b * nkv + kvh) * S * DH;
  const __half *vb = v_cache + (1ll * b * nkv + kvh) * S * DH;
  const bool owns_new = p_new >= p0 && p_new < p1;

  auto load_tile = [&](int t) {
    const int r0 = p0 + t * TP, rows = min(TP, p1 - r0), st = t & 1;
    for (int i = tid; i < rows * VPR; i += kFusedAttnThreads) {
      const int r = i / VPR, c = i - r * VPR;
      if (r0 + r == p_new) continue;  // the new row is not in the cache yet: step 1 puts it here
      cp_async16(smem_u32(ks + (st * TP + r) * KP + 16 * c), kb + 1ll * (r0 + r) * DH + 8 * c);
      cp_async16(smem_u32(vs + (st * TP + r) * VP + 16 * c), vb + 1ll * (r0 + r) * DH + 8 * c);
    }
    cp_async_commit();
  };
  load_tile(0);
  if (ntile > 1) load_tile(1);

  // ---- 1. query heads, new key and value
  const __half *cs = cos_t + p_new * DH, *sn = sin_t + p_new * DH;
  float c0[HALF / 32], s0[HALF / 32], c1[HALF / 32], s1[HALF / 32];
#pragma unroll
  for (int t = 0; t < HALF / 32; ++t) {
    const int i = lane + 32 * t;
    c0[t] = __half2float(cs[i]);
    s0[t] = __half2float(sn[i]);
    c1[t] = __half2float(cs[i + HALF]);
    s1[t] = __half2float(sn[i + HALF]);
  }
  // RMSNorm over the head (when nw), rotary embedding; FP16-rounded results as floats
  auto norm_rope = [&](const float (&x0)[HALF / 32], const float (&x1)[HALF / 32], bool nw, const float (&w0)[HALF / 32],
                       const float (&w1)[HALF / 32], float (&o0)[HALF / 32], float (&o1)[HALF / 32]) {
    float ss = 0.f;
#pragma unroll
    for (int t = 0; t < HALF / 32; ++t) ss += x0[t] * x0[t] + x1[t] * x1[t];
    float rs = 1.f;
    if (nw) rs = rsqrtf(warp_sum(ss) / DH + eps);
#pragma unroll
    for (int t = 0; t < HALF / 32; ++t) {
      float y0 = x0[t], y1 = x1[t];
      if (nw) {
        y0 = __half2float(__hmul(__float2half_rn(x0[t] * rs), __float2half_rn(w0[t])));
        y1 = __half2float(__hmul(__float2half_rn(x1[t] * rs), __float2half_rn(w1[t])));
      }
      o0[t] = __half2float(__float2half_rn(y0 * c0[t] - y1 * s0[t]));
      o1[t] = __half2float(__float2half_rn(y1 * c1[t] + y0 * s1[t]));
    }
  };
  for (int hq = head0; slice == 0 && hq < group; hq += hp) {
    float o0[HALF / 32], o1[HALF / 32];
    if (hq != head0) load_row(row + 1ll * (kvh * group + hq) * DH, qx0, qx1);
    norm_rope(qx0, qx1, qn != nullptr, qw0, qw1, o0, o1);
#pragma unroll
    for (int t = 0; t < HALF / 32; ++t) {
      qs[hq * DH + lane + 32 * t] = o0[t] * scale;
      qs[hq * DH + lane + 32 * t + HALF] = o1[t] * scale;
    }
  }
  // The new row is the last row of the last tile of its CTA.  The last warp (key) and the one
  // before it (value) keep it in registers, write it to the cache now and into the tile when that tile is current.
  float knew0[HALF / 32], knew1[HALF / 32];
  __half vnew[DPL];
  if (owns_new && warp == W - 1) {
    float kx0[HALF / 32], kx1[HALF / 32], kw0[HALF / 32], kw1[HALF / 32];
    load_row(row + 1ll * (nq + kvh) * DH, kx0, kx1);
    if (kn) load_row(kn, kw0, kw1);
    norm_rope(kx0, kx1, kn != nullptr, kw0, kw1, knew0, knew1);
    __half *kd = k_cache + ((1ll * b * nkv + kvh) * S + p_new) * DH;
#pragma unroll
    for (int t = 0; t < HALF / 32; ++t) {
      kd[lane + 32 * t] = __float2half_rn(knew0[t]);
      kd[lane + 32 * t + HALF] = __float2half_rn(knew1[t]);
    }
  }
  if (owns_new && warp == W - 2) {
    const __half *src = row + 1ll * (nq + nkv + kvh) * DH;
    __half *vd = v_cache + ((1ll * b * nkv + kvh) * S + p_new) * DH;
#pragma unroll
    for (int j = 0; j < DPL; ++j) {
      vnew[j] = src[lane + 32 * j];
      vd[lane + 32 * j] = vnew[j];
    }
  }

  // ---- 2./3. tiles
  float m_run[2], l_run[2], acc[2][DPL];  // up to 2 heads per warp (group <= 16)
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    m_run[h] = -INFINITY;
    l_run[h] = 0.f;
#pragma unroll
    for (int j = 0; j < DPL; ++j) acc[h][j] = 0.f;
  }
  for (int t = 0; t < ntile; ++t) {
    if (t + 1 < ntile) cp_async_wait<1>(); else cp_async_wait<0>();
    const int r0 = p0 + t * TP, rows = min(TP, p1 - r0), st = t & 1;
    if (owns_new && t == ntile - 1) {
      const int rr = static_cast<int>(p_new) - r0;
      if (warp == W - 1) {
        __half *sd = reinterpret_cast<__half *>(ks + (st * TP + rr) * KP);
#pragma unroll
        for (int u = 0; u < HALF / 32; ++u) {
          sd[lane + 32 * u] = __float2half_rn(knew0[u]);
          sd[lane + 32 * u + HALF] = __float2half_rn(knew1[u]);
        }
      }
      if (warp == W - 2) {
        __half *sd = reinterpret_cast<__half *>(vs + (st * TP + rr) * VP);
#pragma unroll
        for (int j = 0; j < DPL; ++j) sd[lane + 32 * j] = vnew[j];
      }
    }
    __syncthreads();  // tile t (and, the first time, qs; the last time, the new row) visible to all warps
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int hq = head0 + hp * h;
      if (!active || hq >= group) break;
      const float4 *q4 = reinterpret_cast<const float4 *>(qs + hq * DH);
      for (int rb = 32 * slice; rb < rows; rb += 32 * nsl) {
        const int r = rb + lane;
        float s = -INFINITY;
        if (r < rows) {
          const uint4 *kr = reinterpret_cast<const uint4 *>(ks + (st * TP + r) * KP);
          float d0 = 0.f, d1 = 0.f;
#pragma unroll
          for (int c = 0; c < VPR; ++c) {
            const uint4 kv = kr[c];
            const float4 qa = q4[2 * c], qb = q4[2 * c + 1];
            const float2 k0 = __half22float2(*reinterpret_cast<const __half2 *>(&kv.x));
            const float2 k1 = __half22float2(*reinterpret_cast<const __half2 *>(&kv.y));
            const float2 k2 = __half22float2(*reinterpret_cast<const __half2 *>(&kv.z));
            const float2 k3 = __half22float2(*reinterpret_cast<const __half2 *>(&kv.w));
            d0 += qa.x * k0.x + qa.y * k0.y + qa.z * k1.x + qa.w * k1.y;
            d1 += qb.x * k2.x + qb.y * k2.y + qb.z * k3.x + qb.w * k3.y;
          }
          s = d0 + d1;
        }
        const float mn = fmaxf(m_run[h], warp_max(s));
        const float corr = __expf(m_run[h] - mn);  // 0 the first time (m_run = -inf, mn finite)
        const float w = (r < rows) ? __expf(s - mn) : 0.f;
        l_run[h] = l_run[h] * corr + w;            // per-lane partial sum, reduced at the end
        m_run[h] = mn;
#pragma unroll
        for (int j = 0; j < DPL; ++j) acc[h][j] *= corr;
        const int cnt = min(32, rows - rb);
        const uint8_t *vrow = vs + (st * TP + rb) * VP + lane * DPL * 2;
#pragma unroll 8
        for (int j = 0; j < cnt; ++j) {
          const float wj = __shfl_sync(0xffffffffu, w, j);
          if (DPL == 4) {
            const uint2 v = *reinterpret_cast<const uint2 *>(vrow + j * VP);
            const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&v.x));
            const float2 c = __half22float2(*reinterpret_cast<const __half2 *>(&v.y));
            acc[h][0] += wj * a.x; acc[h][1] += wj * a.y; acc[h][2] += wj * c.x; acc[h][3] += wj * c.y;
          } else {
            const __half *vh = reinterpret_cast<const __half *>(vrow + j * VP);
#pragma unroll
            for (int d = 0; d < DPL; ++d) acc[h][d] += wj * __half2float(vh[d]);
          }
        }
      }
    }
    __syncthreads();  // all warps done with stage st
    if (t + 2 < ntile) load_tile(t + 2);
  }

  // ---- 4. partials: slices above 0 hand theirs to slice 0 through shared memory, slice 0 writes
  // the CTA's partial; merge by the last CTA of this (b, kvh)
#pragma unroll
  for (int h = 0; h < 2; ++h) l_run[h] = warp_sum(l_run[h]);
  if (active && slice > 0) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      if (head0 + hp * h >= group) break;
      float *dst = mrg + (warp * 2 + h) * PR;
      if (lane == 0) {
        dst[0] = m_run[h];
        dst[1] = l_run[h];
      }
#pragma unroll
      for (int j = 0; j < DPL; ++j) dst[4 + lane * DPL + j] = acc[h][j];
    }
  }
  __syncthreads();
  if (slice == 0) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int hq = head0 + hp * h;
      if (hq >= group) break;
      float m = m_run[h];
      for (int sl = 1; sl < nsl; ++sl) m = fmaxf(m, mrg[((sl * hp + head0) * 2 + h) * PR]);
      // (a slice that saw no row has max -inf and weight 0; slice 0 of a CTA with work always has rows)
      const float w0 = __expf(m_run[h] - m);
      float l = l_run[h] * w0;
#pragma unroll
      for (int j = 0; j < DPL; ++j) acc[h][j] *= w0;
      for (int sl = 1; sl < nsl; ++sl) {
        const float *src = mrg + ((sl * hp + head0) * 2 + h) * PR;
        const float ws = __expf(src[0] - m);
        l += src[1] * ws;
#pragma unroll
        for (int j = 0; j < DPL; ++j) acc[h][j] += ws * src[4 + lane * DPL + j];
      }
      float *dst = part + ((1ll * b * nq + kvh * group + hq) * nsplit + split) * PR;
      if (lane == 0) {
        dst[0] = m;
        dst[1] = l;
      }
#pragma unroll
      for (int j = 0; j < DPL; ++j) dst[4 + lane * DPL + j] = acc[h][j];
    }
  }
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const int old = atomicAdd(&counters[b * nkv + kvh], 1);
    s_last = (old == used - 1);
    if (s_last) counters[b * nkv + kvh] = 0;  // ready for the next launch
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // The merging CTA reads `used` partials per head out of L2.  All loads of a batch of splits are
  // issued before any is used (the first batch together with the (max, sum) pairs): two or three
  // round trips per head instead of one per split.
  constexpr int BATCH = 64 / DPL;  // splits per batch: 64 value registers per lane
  for (int hq = warp; hq < group; hq += W) {
    const int head = kvh * group + hq;
    const float *src = part + (1ll * b * nq + head) * nsplit * PR;
    float a[DPL];
#pragma unroll
    for (int j = 0; j < DPL; ++j) a[j] = 0.f;
    float m = 0.f, l = 0.f, w = 0.f;
    for (int s0 = 0; s0 < used; s0 += BATCH) {
      float v[BATCH][DPL];
#pragma unroll
      for (int q = 0; q < BATCH; ++q) {
        if (s0 + q < used) {
          const float *pv = src + (s0 + q) * PR + 4 + lane * DPL;
          if (DPL == 4) {
            const float4 t = __ldcg(reinterpret_cast<const float4 *>(pv));
            v[q][0] = t.x; v[q][1] = t.y; v[q][2] = t.z; v[q][3] = t.w;
          } else {
#pragma unroll
            for (int j = 0; j < DPL; j += 2) {
              const float2 t = __ldcg(reinterpret_cast<const float2 *>(pv + j));
              v[q][j] = t.x; v[q][j + 1] = t.y;
            }
          }
        }
      }
      if (s0 == 0) {  // lane s holds split s's (max, sum); nsplit <= 32
        const float ms = lane < used ? __ldcg(src + lane * PR) : -INFINITY;
        const float ls = lane < used ? __ldcg(src + lane * PR + 1) : 0.f;
        m = warp_max(ms);
        w = lane < used ? __expf(ms - m) : 0.f;
        l = warp_sum(ls * w);
      }
#pragma unroll
      for (int q = 0; q < BATCH; ++q) {
        if (s0 + q < used) {
          const float ws = __shfl_sync(0xffffffffu, w, s0 + q);
#pragma unroll
          for (int j = 0; j < DPL; ++j) a[j] += ws * v[q][j];
        }
      }
    }
    __half *o = out + (1ll * b * nq + head) * DH + lane * DPL;
    const float inv = 1.f / l;
#pragma unroll
    for (int j = 0; j < DPL; ++j) o[j] = __float2half_rn(a[j] * inv);
  }
}

// `slot`: the kernel sits between two GEMVs of a decode step: it reserves kSlotSmem of (unused)
// shared memory so that no SM takes two of its CTAs (see pin_slot).
template <typename... Args>
int launch_pdl(void (*kernel)(Args...), dim3 grid, dim3 block, bool slot, bool pdl, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = slot ? kSlotSmem : 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (slot) RDQ_CUDA(pin_slot(reinterpret_cast<const void *>(kernel), kSlotSmem));
  RDQ_CUDA(cudaLaunchKernelEx(&cfg, kernel, args...));
  return RDQ_OK;
}

}  // namespace

// An SM cannot change its shared-memory carve-out while a CTA is resident, and the kernels of a
// decode step overlap on every SM: all of them ask for the largest carve-out, like the GEMV.
// `smem` is the dynamic shared memory the kernel will be launched with.  Once per kernel, device
// and size.
cudaError_t pin_slot(const void *fn, int smem) {
  static std::mutex mu;
  static std::vector<std::pair<std::pair<const void *, int>, int>> done;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  std::lock_guard<std::mutex> lock(mu);
  for (const auto &d : done)
    if (d.first.first == fn && d.first.second == dev && d.second >= smem) return cudaSuccess;
  e = cudaFuncSetAttribute(fn, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  if (e == cudaSuccess && smem > 48 * 1024) e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e == cudaSuccess) done.push_back({{fn, dev}, smem});
  return e;
}

int launch_add_rmsnorm(__half *x, const __half *delta, const __half *w, __half *out, int B, int H, float eps, bool pdl,
                       cudaStream_t stream) {
  return launch_pdl(add_rmsnorm_kernel, dim3(std::max(B, sm_count())), dim3(256), true, pdl, stream, x, delta, w, out, B, H, eps);
}

int launch_qk_rope_cache(const __half *qkv, const __half *qn, const __half *kn, const __half *cos_t, const __half *sin_t,
                         const long long *pos, __half *q_out, __half *k_cache, __half *v_cache, int B, int nq, int nkv,
                         int dh, int S, float eps, bool pdl, cudaStream_t stream) {
  return launch_pdl(qk_rope_cache_kernel, dim3(nq + 2 * nkv, B), dim3(dh / 2), false, pdl, stream, qkv, qn, kn, cos_t, sin_t, pos,
                    q_out, k_cache, v_cache, nq, nkv, dh, S, eps);
}

int attn_chunk() { return 32; }

int launch_attn_decode(const __half *q, const __half *k_cache, const __half *v_cache, const long long *pos, float *scratch,
                       __half *out, int B, int nq, int nkv, int dh, int S, float scale, bool pdl, cudaStream_t stream) {
  const int chunk = attn_chunk();
  const int nsplit = (S + chunk - 1) / chunk;
  int rc = launch_pdl(attn_split_kernel, dim3(nsplit, nkv, B), dim3(kAttnWarps * 32), false, pdl, stream, q, k_cache, v_cache, pos,
                      scratch, nq, nkv, dh, S, chunk, scale);
  if (rc != RDQ_OK) return rc;
  return launch_pdl(attn_combine_kernel, dim3(nq, B), dim3(dh), false, pdl, stream, static_cast<const float *>(scratch), out, nq, dh,
                    nsplit);
}

// Splits of the cache rows per (sequence, KV head): as many as give every SM one CTA.
int rope_attn_splits(int B, int nkv, int S) {
  (void)S;
  return std::min(kFusedAttnMaxSplit, std::max(1, sm_count() / std::max(1, B * nkv)));
}

size_t rope_attn_scratch_bytes(int B, int nq, int nkv, int dh, int S) {
  // counters first (4-byte ints, rounded up to 256 bytes), then the partials.  Sized for every
  // batch up to B (fewer sequences get more splits each), so one buffer serves smaller batches.
  const size_t cnt = (static_cast<size_t>(B) * nkv * sizeof(int) + 255) & ~static_cast<size_t>(255);
  size_t rows = 0;
  for (int b = 1; b <= B; ++b) rows = std::max(rows, static_cast<size_t>(b) * rope_attn_splits(b, nkv, S));
  return cnt + sizeof(float) * rows * nq * (dh + 4);
}

int launch_rope_attn(const __half *qkv, const __half *qn, const __half *kn, const __half *cos_t, const __half *sin_t,
                     const long long *pos, __half *k_cache, __half *v_cache, void *scratch, __half *out, int B, int nq,
                     int nkv, int dh, int S, float scale, float eps, bool pdl, cudaStream_t stream) {
  const int nsplit = rope_attn_splits(B, nkv, S);
  const size_t cnt = (static_cast<size_t>(B) * nkv * sizeof(int) + 255) & ~static_cast<size_t>(255);
  int *counters = static_cast<int *>(scratch);
  float *part = reinterpret_cast<float *>(static_cast<uint8_t *>(scratch) + cnt);
  const int group = nq / nkv;
  const int tp = 8192 / dh;
  const int smem = 2 * tp * (2 * dh + 16) + 2 * tp * 2 * dh + group * dh * 4 + kFusedAttnWarps * 2 * (dh + 4) * 4;
  auto launch = [&](auto kernel) -> int {
    cudaLaunchConfig_t cfg = {};
    // one CTA per SM while the (sequence, KV head) pairs fit: like the GEMVs around it
    cfg.gridDim = dim3(std::max(sm_count(), nsplit * nkv * B));
    cfg.blockDim = dim3(kFusedAttnThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = pdl ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    RDQ_CUDA(pin_slot(reinterpret_cast<const void *>(kernel), smem));
    RDQ_CUDA(cudaLaunchKernelEx(&cfg, kernel, qkv, qn, kn, cos_t, sin_t, pos, k_cache, v_cache, part, counters, out, nq, nkv, S,
                                scale, eps, nsplit, nkv * B));
    return RDQ_OK;
  };
  switch (dh) {
    case 64: return launch(rope_attn_kernel<64>);
    case 128: return launch(rope_attn_kernel<128>);
    case 256: return launch(rope_attn_kernel<256>);
  }
  RDQ_REQUIRE(false, RDQ_E_UNSUPPORTED, "head_dim must be 64, 128 or 256, got %d", dh);
  return RDQ_OK;
}

int launch_silu_mul(const __half *gu, __half *out, int B, int F, bool pdl, cudaStream_t stream) {
  const long long total = 1ll * B * (F / 8);
  (void)total;
  return launch_pdl(silu_mul_kernel, dim3(sm_count()), dim3(256), true, pdl, stream, gu, out, B, F);
}

}  // namespace rdq
