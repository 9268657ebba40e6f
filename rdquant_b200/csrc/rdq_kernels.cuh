// Internal launch interfaces shared by the C-ABI translation unit and the
// kernel translation units.
#pragma once

#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <mutex>

#include "rdq_common.cuh"

namespace rdq {

constexpr int kMaxPeers = 8;  // GPUs of one node a peer-mode launch can write to

// Arguments of the decode GEMV kernels (permuted-row tensors, see rdq_b200.h).
struct GemvArgs {
  const __half *x;
  int M;
  const uint8_t *w4;
  const uint8_t *s4;
  float global4;
  const uint8_t *w8;
  const float *s8;
  const __half *w16;
  const int32_t *perm;
  const __half *bias;
  __half *y;
  int n4, n8, n16, K;
  float *workspace;   // unused by the any-shape kernel
  int32_t *counters;
};

struct GemmArgs {
  const __half *x;
  int M;
  const uint8_t *w4;
  const uint8_t *s4;
  float global4;
  const uint8_t *w8;
  const float *s8;
  const __half *w16;
  const int32_t *inv_perm;
  const __half *bias;
  __half *y;
  int n4, n8, n16, K;
  int ksplit;      // CTAs that share the k range of a tile (blockIdx.z); 1 = no split
  float *partial;  // ksplit > 1: raw FP32 sums [ksplit][M][N], reduced by a second kernel
  int test_timeout = 0;  // self-test: CTA (0,0,0) ends with a wait that runs out
};

int launch_dequant(const void *w_fp4, const void *w_fp4_scales, float global4, const void *w_fp8,
                   const float *w_fp8_scales, const void *w_fp16, int fp16_is_bf16,
                   const int32_t *inv_perm, void *w_out, int out_is_f32, int n4, int n8, int n16,
                   int K, cudaStream_t stream);

int launch_gemv_generic(const GemvArgs &a, cudaStream_t stream);

// ---- tiled layout (rdq_gemv_tiled.cu)
struct GemvTiledArgs {
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
  int32_t *flags;
  int test_timeout = 0;  // RDQ_GEMV_TEST_TIMEOUT
  // peer mode (see TiledArgs): destinations, this rank's flag word on every GPU, local state
  int n_dst = 0;
  __half *dst[kMaxPeers] = {};
  int32_t *peer_flag[kMaxPeers] = {};
  int32_t *peer_state = nullptr;
  // activation prologue (see TiledArgs)
  int xop = 0;
  const __half *x_aux = nullptr;
  const __half *x_weight = nullptr;
  __half *x_out = nullptr;
  float x_eps = 0.f;
};
int tiled_chunk_k(int K);
// true when the launcher keeps the activation rows of this shape in shared memory (a requirement
// of the activation prologue)
bool tiled_stages_x(int M, int K);
bool tiled_supported(int n4, int n8, int n16, int K);
size_t tiled_bytes(int n4, int n8, int n16, int K);
int launch_repack(const void *w_fp4, const void *w_fp4_scales, const void *w_fp8, const void *w_fp16,
                  void *tiled_out, int n4, int n8, int n16, int K, cudaStream_t stream);
void gemv_tiled_scratch(size_t *workspace_bytes, size_t *flag_bytes);
int launch_gemv_tiled(const GemvTiledArgs &a, bool pdl, cudaStream_t stream);
// same kernel with the scratch in a library-owned device array (no allocation anywhere)
int gemv_tiled_noalloc(const GemvTiledArgs &a, bool pdl, cudaStream_t stream);
// synchronise `stream`, report (and optionally clear) the kernel's status word; null scratch
// pointers select the library array of the no-allocation entry point
int gemv_tiled_status(float *workspace, int32_t *flags, bool reset, cudaStream_t stream);
int launch_peer_gather(const __half *buffer, const long long *index, __half *y, long long count, const int32_t *flags,
                       int world, const int32_t *sent_state, int32_t *status, int wait_ms, bool pdl, cudaStream_t stream);

int launch_gemm(const GemmArgs &a, void *workspace, size_t workspace_bytes, cudaStream_t stream);
// synchronise `stream`, report (and optionally clear) the GEMM's per-device status word
int gemm_status(bool reset, cudaStream_t stream);
// self-test switch: launches made while it is on end with a wait that runs out
void gemm_set_test_timeout(bool on);
size_t gemm_workspace_bytes(int M, int N, int K);

// staging copy by kernel (rdq_stage.cu)
int launch_stage_copy(void *dst, const void *src, size_t bytes, int *state, int *flag, cudaStream_t stream);

// decode-step glue (rdq_glue.cu)
int launch_add_rmsnorm(__half *x, const __half *delta, const __half *w, __half *out, int B, int H, float eps, bool pdl,
                       cudaStream_t stream);
int launch_qk_rope_cache(const __half *qkv, const __half *qn, const __half *kn, const __half *cos_t, const __half *sin_t,
                         const long long *pos, __half *q_out, __half *k_cache, __half *v_cache, int B, int nq, int nkv,
                         int dh, int S, float eps, bool pdl, cudaStream_t stream);
// Kernels that sit between two GEMVs of a decode step are launched with one CTA per SM and this
// much (unused) dynamic shared memory: next to a GEMV's CTA (<= 112 KB + static) an SM then has
// room for one of their CTAs, not two.
constexpr int kSlotSmem = 60 * 1024;
cudaError_t pin_slot(const void *fn, int smem);
int attn_chunk();
// q/k norm + rotary + cache write + attention + merge of the splits in one launch
int rope_attn_splits(int B, int nkv, int S);
size_t rope_attn_scratch_bytes(int B, int nq, int nkv, int dh, int S);
int launch_rope_attn(const __half *qkv, const __half *qn, const __half *kn, const __half *cos_t, const __half *sin_t,
                     const long long *pos, __half *k_cache, __half *v_cache, void *scratch, __half *out, int B, int nq,
                     int nkv, int dh, int S, float scale, float eps, bool pdl, cudaStream_t stream);
int launch_attn_decode(const __half *q, const __half *k_cache, const __half *v_cache, const long long *pos, float *scratch,
                       __half *out, int B, int nq, int nkv, int dh, int S, float scale, bool pdl, cudaStream_t stream);
int launch_silu_mul(const __half *gu, __half *out, int B, int F, bool pdl, cudaStream_t stream);

// encoders (rdq_quantize.cu)
int launch_quantize_nvfp4(const void *w, bool w_is_f32, int n, int K, uint8_t *codes, uint8_t *scales, float *row_sqerr,
                          float *max_scale, cudaStream_t stream);
int launch_quantize_fp8(const void *w, bool w_is_f32, int n, int K, uint8_t *out, float *scale_out, float *row_sqerr,
                        float *absmax_scratch, cudaStream_t stream);

}  // namespace rdq
