// C ABI of librdq_b200.so: argument validation and dispatch to the kernels.
// Declarations and the reference interfaces they replace: include/rdq_b200.h.
#include <cstdarg>
#include <cstring>

#include "rdq_kernels.cuh"

namespace rdq {

static thread_local char g_error[512] = "";

void set_error(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

int sm_count() {
  static std::atomic<int> cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 1;
  if (dev >= 0 && dev < 64 && cached[dev].load() > 0) return cached[dev].load();
  int n = 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 1;
  if (dev >= 0 && dev < 64) cached[dev].store(n);
  return n;
}

namespace {

// Shape / pointer checks shared by the three operators; mirrors the
// TORCH_CHECKs of the reference wrapper (rdquant/csrc/bindings.cpp:167-182).
int check_layer(const void *w_fp4, const void *w_fp4_scales, const void *w_fp8,
                const float *w_fp8_scales, const void *w_fp16, int n4, int n8, int n16, int K) {
  RDQ_REQUIRE(n4 >= 0 && n8 >= 0 && n16 >= 0, RDQ_E_INVALID, "group sizes must be non-negative");
  RDQ_REQUIRE(K > 0, RDQ_E_INVALID, "K must be positive");
  if (n4 > 0) {
    RDQ_REQUIRE(K % 16 == 0, RDQ_E_INVALID,
                "NVFP4 group needs K to be a multiple of 16 (one E4M3 scale per 16 k), got K=%d", K);
    RDQ_REQUIRE(w_fp4 && w_fp4_scales, RDQ_E_INVALID, "w_fp4 / w_fp4_scales must not be null when n_fp4 > 0");
    RDQ_REQUIRE(aligned16(w_fp4) && aligned16(w_fp4_scales), RDQ_E_INVALID,
                "w_fp4 / w_fp4_scales must be 16-byte aligned");
  }
  if (n8 > 0) {
    RDQ_REQUIRE(w_fp8 && w_fp8_scales, RDQ_E_INVALID, "w_fp8 / w_fp8_scales must not be null when n_fp8 > 0");
    RDQ_REQUIRE(aligned16(w_fp8), RDQ_E_INVALID, "w_fp8 must be 16-byte aligned");
  }
  if (n16 > 0) {
    RDQ_REQUIRE(w_fp16 != nullptr, RDQ_E_INVALID, "w_fp16 must not be null when n_fp16 > 0");
    RDQ_REQUIRE(aligned16(w_fp16), RDQ_E_INVALID, "w_fp16 must be 16-byte aligned");
  }
  return RDQ_OK;
}

}  // namespace
}  // namespace rdq

using namespace rdq;

extern "C" {

int rdq_version(void) { return 100; }

const char *rdq_last_error(void) { return g_error; }

int rdq_dequant_packed(const void *w_fp4, const void *w_fp4_scales, float w_fp4_global_scale,
                       const void *w_fp8, const float *w_fp8_scales, const void *w_fp16,
                       int fp16_is_bf16, const int32_t *inv_perm, void *w_out, int out_is_f32,
                       int n_fp4, int n_fp8, int n_fp16, int K, void *stream) {
  int rc = check_layer(w_fp4, w_fp4_scales, w_fp8, w_fp8_scales, w_fp16, n_fp4, n_fp8, n_fp16, K);
  if (rc != RDQ_OK) return rc;
  if (n_fp4 + n_fp8 + n_fp16 == 0) return RDQ_OK;
  RDQ_REQUIRE(w_out != nullptr && aligned16(w_out), RDQ_E_INVALID, "w_out must be a 16-byte aligned device pointer");
  return launch_dequant(w_fp4, w_fp4_scales, w_fp4_global_scale, w_fp8, w_fp8_scales, w_fp16,
                        fp16_is_bf16, inv_perm, w_out, out_is_f32, n_fp4, n_fp8, n_fp16, K,
                        static_cast<cudaStream_t>(stream));
}

int rdq_gemv_scratch_size(int N, size_t *workspace_bytes, size_t *counter_bytes) {
  RDQ_REQUIRE(N >= 0 && workspace_bytes && counter_bytes, RDQ_E_INVALID, "bad arguments to rdq_gemv_scratch_size");
  (void)N;
  gemv_tiled_scratch(workspace_bytes, counter_bytes);
  return RDQ_OK;
}

int rdq_gemv_mixed(const void *x, int M, const void *w_fp4, const void *w_fp4_scales,
                   float w_fp4_global_scale, const void *w_fp8, const float *w_fp8_scales,
                   const void *w_fp16, const int32_t *perm, const void *bias, void *y, int n_fp4,
                   int n_fp8, int n_fp16, int K, void *workspace, int32_t *counters, int flags,
                   void *stream) {
  int rc = check_layer(w_fp4, w_fp4_scales, w_fp8, w_fp8_scales, w_fp16, n_fp4, n_fp8, n_fp16, K);
  if (rc != RDQ_OK) return rc;
  RDQ_REQUIRE(M >= 0 && M <= RDQ_MAX_GEMV_M, RDQ_E_UNSUPPORTED,
              "rdq_gemv_mixed takes 1..%d activation rows, got M=%d (use rdq_gemm_mixed)", RDQ_MAX_GEMV_M, M);
  if (M == 0 || n_fp4 + n_fp8 + n_fp16 == 0) return RDQ_OK;
  RDQ_REQUIRE(x != nullptr && y != nullptr, RDQ_E_INVALID, "x and y must not be null");
  RDQ_REQUIRE(aligned16(x) || (K % 16 != 0), RDQ_E_INVALID, "x must be 16-byte aligned");
  GemvArgs a;
  a.x = static_cast<const __half *>(x);
  a.M = M;
  a.w4 = static_cast<const uint8_t *>(w_fp4);
  a.s4 = static_cast<const uint8_t *>(w_fp4_scales);
  a.global4 = w_fp4_global_scale;
  a.w8 = static_cast<const uint8_t *>(w_fp8);
  a.s8 = w_fp8_scales;
  a.w16 = static_cast<const __half *>(w_fp16);
  a.perm = perm;
  a.bias = static_cast<const __half *>(bias);
  a.y = static_cast<__half *>(y);
  a.n4 = n_fp4;
  a.n8 = n_fp8;
  a.n16 = n_fp16;
  a.K = K;
  a.workspace = static_cast<float *>(workspace);
  a.counters = counters;
  (void)flags;
  return launch_gemv_generic(a, static_cast<cudaStream_t>(stream));
}

size_t rdq_gemv_tiled_bytes(int n_fp4, int n_fp8, int n_fp16, int K) {
  if (n_fp4 < 0 || n_fp8 < 0 || n_fp16 < 0 || !tiled_supported(n_fp4, n_fp8, n_fp16, K)) return 0;
  return tiled_bytes(n_fp4, n_fp8, n_fp16, K);
}

int rdq_gemv_repack(const void *w_fp4, const void *w_fp4_scales, const void *w_fp8, const void *w_fp16,
                    void *w_tiled, int n_fp4, int n_fp8, int n_fp16, int K, void *stream) {
  int rc = check_layer(w_fp4, w_fp4_scales, w_fp8, reinterpret_cast<const float *>(w_fp8), w_fp16, n_fp4, n_fp8,
                       n_fp16, K);
  if (rc != RDQ_OK) return rc;
  RDQ_REQUIRE(tiled_supported(n_fp4, n_fp8, n_fp16, K), RDQ_E_UNSUPPORTED,
              "tiled layout needs groups in multiples of 16 rows and K divisible into chunks that are "
              "multiples of 64 (K=%d, n=%d/%d/%d)", K, n_fp4, n_fp8, n_fp16);
  RDQ_REQUIRE(w_tiled != nullptr && aligned16(w_tiled), RDQ_E_INVALID, "w_tiled must be a 16-byte aligned device pointer");
  return launch_repack(w_fp4, w_fp4_scales, w_fp8, w_fp16, w_tiled, n_fp4, n_fp8, n_fp16, K,
                       static_cast<cudaStream_t>(stream));
}

int rdq_gemv_tiled(const void *x, int M, const void *w_tiled, const float *w_fp8_scales, float w_fp4_global_scale,
                   const int32_t *perm, const void *bias, void *y, int n_fp4, int n_fp8, int n_fp16, int K,
                   void *workspace, int32_t *counters, int flags, void *stream) {
  RDQ_REQUIRE(n_fp4 >= 0 && n_fp8 >= 0 && n_fp16 >= 0 && K > 0, RDQ_E_INVALID, "bad layer shape");
  RDQ_REQUIRE(M >= 0 && M <= RDQ_MAX_GEMV_M, RDQ_E_UNSUPPORTED,
              "rdq_gemv_tiled takes 1..%d activation rows, got M=%d (use rdq_gemm_mixed)", RDQ_MAX_GEMV_M, M);
  if (M == 0 || n_fp4 + n_fp8 + n_fp16 == 0) return RDQ_OK;
  RDQ_REQUIRE(tiled_supported(n_fp4, n_fp8, n_fp16, K), RDQ_E_UNSUPPORTED,
              "shape has no tiled layout (K=%d, n=%d/%d/%d)", K, n_fp4, n_fp8, n_fp16);
  RDQ_REQUIRE(x && y && w_tiled && workspace && counters, RDQ_E_INVALID,
              "x, y, w_tiled, workspace and counters must not be null");
  RDQ_REQUIRE(aligned16(x) && aligned16(w_tiled), RDQ_E_INVALID, "x and w_tiled must be 16-byte aligned");
  RDQ_REQUIRE(n_fp8 == 0 || w_fp8_scales != nullptr, RDQ_E_INVALID, "w_fp8_scales must not be null when n_fp8 > 0");
  GemvTiledArgs a;
  a.x = static_cast<const __half *>(x);
  a.M = M;
  a.tiled = static_cast<const uint8_t *>(w_tiled);
  a.s8 = w_fp8_scales;
  a.global4 = w_fp4_global_scale;
  a.perm = perm;
  a.bias = static_cast<const __half *>(bias);
  a.y = static_cast<__half *>(y);
  a.n4 = n_fp4;
  a.n8 = n_fp8;
  a.n16 = n_fp16;
  a.K = K;
  a.workspace = static_cast<float *>(workspace);
  a.flags = counters;
  a.test_timeout = (flags & RDQ_GEMV_TEST_TIMEOUT) ? 1 : 0;
  return launch_gemv_tiled(a, (flags & RDQ_GEMV_PDL) != 0, static_cast<cudaStream_t>(stream));
}

int rdq_gemv_tiled_stages_x(int M, int K) { return (K > 0 && K % 128 == 0 && tiled_stages_x(M, K)) ? 1 : 0; }
int rdq_gemv_tiled_xop(int op, const void *x, const void *x_aux, const void *x_weight, void *x_out, float eps, int M,
                       const void *w_tiled, const float *w_fp8_scales, float w_fp4_global_scale, const int32_t *perm,
                       const void *bias, void *y, int n_fp4, int n_fp8, int n_fp16, int K, void *workspace,
                       int32_t *counters, int flags, void *stream) {
  RDQ_REQUIRE(op == RDQ_XOP_ADD_RMSNORM || op == RDQ_XOP_SILU_MUL, RDQ_E_INVALID, "unknown activation prologue %d", op);
  RDQ_REQUIRE(n_fp4 >= 0 && n_fp8 >= 0 && n_fp16 >= 0 && K > 0, RDQ_E_INVALID, "bad layer shape");
  RDQ_REQUIRE(M >= 1 && M <= RDQ_MAX_GEMV_M, RDQ_E_UNSUPPORTED, "rdq_gemv_tiled_xop takes 1..%d activation rows, got M=%d",
              RDQ_MAX_GEMV_M, M);
  if (n_fp4 + n_fp8 + n_fp16 == 0) return RDQ_OK;
  RDQ_REQUIRE(tiled_supported(n_fp4, n_fp8, n_fp16, K), RDQ_E_UNSUPPORTED,
              "shape has no tiled layout (K=%d, n=%d/%d/%d)", K, n_fp4, n_fp8, n_fp16);
  RDQ_REQUIRE(x && y && w_tiled && workspace && counters, RDQ_E_INVALID,
              "x, y, w_tiled, workspace and counters must not be null");
  RDQ_REQUIRE(aligned16(x) && aligned16(w_tiled) && aligned16(x_aux) && aligned16(x_weight) && aligned16(x_out),
              RDQ_E_INVALID, "x, x_aux, x_weight, x_out and w_tiled must be 16-byte aligned");
  RDQ_REQUIRE(op != RDQ_XOP_ADD_RMSNORM || x_weight != nullptr, RDQ_E_INVALID, "x_weight must not be null");
  RDQ_REQUIRE(x_out == nullptr || (x_out != x && x_out != x_aux), RDQ_E_INVALID,
              "x_out must not alias x or x_aux: every CTA reads them");
  RDQ_REQUIRE(n_fp8 == 0 || w_fp8_scales != nullptr, RDQ_E_INVALID, "w_fp8_scales must not be null when n_fp8 > 0");
  GemvTiledArgs a;
  a.x = static_cast<const __half *>(x);
  a.M = M;
  a.tiled = static_cast<const uint8_t *>(w_tiled);
  a.s8 = w_fp8_scales;
  a.global4 = w_fp4_global_scale;
  a.perm = perm;
  a.bias = static_cast<const __half *>(bias);
  a.y = static_cast<__half *>(y);
  a.n4 = n_fp4;
  a.n8 = n_fp8;
  a.n16 = n_fp16;
  a.K = K;
  a.workspace = static_cast<float *>(workspace);
  a.flags = counters;
  a.test_timeout = 0;
  a.xop = op;
  if (op == RDQ_XOP_ADD_RMSNORM) {
    a.x_aux = static_cast<const __half *>(x_aux);
    a.x_weight = static_cast<const __half *>(x_weight);
    a.x_out = static_cast<__half *>(x_out);
    a.x_eps = eps;
  }
  return launch_gemv_tiled(a, (flags & RDQ_GEMV_PDL) != 0, static_cast<cudaStream_t>(stream));
}
int rdq_gemv_tiled_peer(const void *x, int M, const void *w_tiled, const float *w_fp8_scales, float w_fp4_global_scale,
                        const int32_t *perm, const void *bias, void *const *dst, int32_t *const *peer_flags, int n_dst,
                        int32_t *peer_state, int n_fp4, int n_fp8, int n_fp16, int K, void *workspace, int32_t *counters,
                        int flags, void *stream) {
  RDQ_REQUIRE(n_fp4 >= 0 && n_fp8 >= 0 && n_fp16 >= 0 && K > 0, RDQ_E_INVALID, "bad layer shape");
  RDQ_REQUIRE(M >= 1 && M <= RDQ_MAX_GEMV_M, RDQ_E_UNSUPPORTED, "rdq_gemv_tiled_peer takes 1..%d activation rows, got M=%d",
              RDQ_MAX_GEMV_M, M);
  RDQ_REQUIRE(n_dst >= 1 && n_dst <= kMaxPeers, RDQ_E_UNSUPPORTED, "1..%d destinations, got %d", kMaxPeers, n_dst);
  RDQ_REQUIRE(tiled_supported(n_fp4, n_fp8, n_fp16, K), RDQ_E_UNSUPPORTED, "shape has no tiled layout (K=%d, n=%d/%d/%d)", K,
              n_fp4, n_fp8, n_fp16);
  RDQ_REQUIRE(x && w_tiled && workspace && counters && dst && peer_flags && peer_state, RDQ_E_INVALID, "null pointer");
  RDQ_REQUIRE(aligned16(x) && aligned16(w_tiled), RDQ_E_INVALID, "x and w_tiled must be 16-byte aligned");
  RDQ_REQUIRE(n_fp8 == 0 || w_fp8_scales != nullptr, RDQ_E_INVALID, "w_fp8_scales must not be null when n_fp8 > 0");
  GemvTiledArgs a;
  a.x = static_cast<const __half *>(x);
  a.M = M;
  a.tiled = static_cast<const uint8_t *>(w_tiled);
  a.s8 = w_fp8_scales;
  a.global4 = w_fp4_global_scale;
  a.perm = perm;
  a.bias = static_cast<const __half *>(bias);
  a.y = nullptr;
  a.n4 = n_fp4;
  a.n8 = n_fp8;
  a.n16 = n_fp16;
  a.K = K;
  a.workspace = static_cast<float *>(workspace);
  a.flags = counters;
  a.test_timeout = 0;
  a.n_dst = n_dst;
  for (int d = 0; d < n_dst; ++d) {
    RDQ_REQUIRE(dst[d] != nullptr && peer_flags[d] != nullptr, RDQ_E_INVALID, "destination %d is null", d);
    a.dst[d] = static_cast<__half *>(dst[d]);
    a.peer_flag[d] = peer_flags[d];
  }
  a.peer_state = peer_state;
  return launch_gemv_tiled(a, (flags & RDQ_GEMV_PDL) != 0, static_cast<cudaStream_t>(stream));
}

int rdq_peer_gather(const void *buffer, const long long *index, void *y, long long count, const int32_t *flags, int world,
                    const int32_t *peer_state, int32_t *status, int wait_ms, int flags_pdl, void *stream) {
  RDQ_REQUIRE(count >= 0 && world >= 1 && world <= kMaxPeers && wait_ms > 0, RDQ_E_INVALID, "bad arguments to rdq_peer_gather");
  RDQ_REQUIRE(buffer && index && y && flags && peer_state && status, RDQ_E_INVALID, "null pointer");
  return launch_peer_gather(static_cast<const __half *>(buffer), index, static_cast<__half *>(y), count, flags, world,
                            peer_state, status, wait_ms, (flags_pdl & RDQ_GEMV_PDL) != 0, static_cast<cudaStream_t>(stream));
}

int rdq_gemv_tiled_noalloc(const void *x, int M, const void *w_tiled, const float *w_fp8_scales,
                           float w_fp4_global_scale, const int32_t *perm, const void *bias, void *y, int n_fp4,
                           int n_fp8, int n_fp16, int K, int flags, void *stream) {
  RDQ_REQUIRE(n_fp4 >= 0 && n_fp8 >= 0 && n_fp16 >= 0 && K > 0, RDQ_E_INVALID, "bad layer shape");
  RDQ_REQUIRE(M >= 0 && M <= RDQ_MAX_GEMV_M, RDQ_E_UNSUPPORTED,
              "rdq_gemv_tiled_noalloc takes 1..%d activation rows, got M=%d", RDQ_MAX_GEMV_M, M);
  if (M == 0 || n_fp4 + n_fp8 + n_fp16 == 0) return RDQ_OK;
  RDQ_REQUIRE(tiled_supported(n_fp4, n_fp8, n_fp16, K), RDQ_E_UNSUPPORTED,
              "shape has no tiled layout (K=%d, n=%d/%d/%d)", K, n_fp4, n_fp8, n_fp16);
  RDQ_REQUIRE(x && y && w_tiled, RDQ_E_INVALID, "x, y and w_tiled must not be null");
  RDQ_REQUIRE(aligned16(x) && aligned16(w_tiled), RDQ_E_INVALID, "x and w_tiled must be 16-byte aligned");
  RDQ_REQUIRE(n_fp8 == 0 || w_fp8_scales != nullptr, RDQ_E_INVALID, "w_fp8_scales must not be null when n_fp8 > 0");
  GemvTiledArgs a;
  a.x = static_cast<const __half *>(x);
  a.M = M;
  a.tiled = static_cast<const uint8_t *>(w_tiled);
  a.s8 = w_fp8_scales;
  a.global4 = w_fp4_global_scale;
  a.perm = perm;
  a.bias = static_cast<const __half *>(bias);
  a.y = static_cast<__half *>(y);
  a.n4 = n_fp4;
  a.n8 = n_fp8;
  a.n16 = n_fp16;
  a.K = K;
  a.workspace = nullptr;
  a.flags = nullptr;
  a.test_timeout = (flags & RDQ_GEMV_TEST_TIMEOUT) ? 1 : 0;
  return gemv_tiled_noalloc(a, (flags & RDQ_GEMV_PDL) != 0, static_cast<cudaStream_t>(stream));
}

int rdq_gemv_tiled_status(void *workspace, int32_t *counters, int reset, void *stream) {
  RDQ_REQUIRE(workspace != nullptr && counters != nullptr, RDQ_E_INVALID, "workspace and counters must not be null");
  return gemv_tiled_status(static_cast<float *>(workspace), counters, reset != 0, static_cast<cudaStream_t>(stream));
}

int rdq_gemv_tiled_noalloc_status(int reset, void *stream) {
  return gemv_tiled_status(nullptr, nullptr, reset != 0, static_cast<cudaStream_t>(stream));
}

int rdq_gemm_status(int reset, void *stream) { return gemm_status(reset != 0, static_cast<cudaStream_t>(stream)); }

void rdq_gemm_test_timeout(int enable) { gemm_set_test_timeout(enable != 0); }

int rdq_gemm_mixed_ws(const void *x, int M, const void *w_fp4, const void *w_fp4_scales,
                      float w_fp4_global_scale, const void *w_fp8, const float *w_fp8_scales,
                      const void *w_fp16, const int32_t *inv_perm, const void *bias, void *y, int n_fp4,
                      int n_fp8, int n_fp16, int K, void *workspace, size_t workspace_bytes, void *stream) {
  int rc = check_layer(w_fp4, w_fp4_scales, w_fp8, w_fp8_scales, w_fp16, n_fp4, n_fp8, n_fp16, K);
  if (rc != RDQ_OK) return rc;
  RDQ_REQUIRE(M >= 0, RDQ_E_INVALID, "M must be non-negative");
  if (M == 0 || n_fp4 + n_fp8 + n_fp16 == 0) return RDQ_OK;
  RDQ_REQUIRE(x != nullptr && y != nullptr, RDQ_E_INVALID, "x and y must not be null");
  RDQ_REQUIRE(aligned16(x) && aligned16(y), RDQ_E_INVALID, "x and y must be 16-byte aligned");
  RDQ_REQUIRE(K % 64 == 0, RDQ_E_UNSUPPORTED, "rdq_gemm_mixed needs K to be a multiple of 64, got K=%d", K);
  // the kernel addresses each weight tensor with 32-bit byte offsets
  RDQ_REQUIRE(1ll * n_fp4 * (K / 2) < (1ll << 32) && 1ll * n_fp8 * K < (1ll << 32) && 2ll * n_fp16 * K < (1ll << 32),
              RDQ_E_UNSUPPORTED, "rdq_gemm_mixed: a format group of this layer exceeds 4 GB");
  GemmArgs a;
  a.x = static_cast<const __half *>(x);
  a.M = M;
  a.w4 = static_cast<const uint8_t *>(w_fp4);
  a.s4 = static_cast<const uint8_t *>(w_fp4_scales);
  a.global4 = w_fp4_global_scale;
  a.w8 = static_cast<const uint8_t *>(w_fp8);
  a.s8 = w_fp8_scales;
  a.w16 = static_cast<const __half *>(w_fp16);
  a.inv_perm = inv_perm;
  a.bias = static_cast<const __half *>(bias);
  a.y = static_cast<__half *>(y);
  a.n4 = n_fp4;
  a.n8 = n_fp8;
  a.n16 = n_fp16;
  a.K = K;
  a.ksplit = 1;
  a.partial = nullptr;
  RDQ_REQUIRE(workspace == nullptr || aligned16(workspace), RDQ_E_INVALID, "workspace must be 16-byte aligned");
  return launch_gemm(a, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

int rdq_gemm_mixed(const void *x, int M, const void *w_fp4, const void *w_fp4_scales,
                   float w_fp4_global_scale, const void *w_fp8, const float *w_fp8_scales,
                   const void *w_fp16, const int32_t *inv_perm, const void *bias, void *y, int n_fp4,
                   int n_fp8, int n_fp16, int K, void *stream) {
  return rdq_gemm_mixed_ws(x, M, w_fp4, w_fp4_scales, w_fp4_global_scale, w_fp8, w_fp8_scales, w_fp16, inv_perm, bias, y,
                           n_fp4, n_fp8, n_fp16, K, nullptr, 0, stream);
}

int rdq_gemm_workspace_size(int M, int N, int K, size_t *bytes) {
  RDQ_REQUIRE(bytes != nullptr, RDQ_E_INVALID, "bytes must not be null");
  RDQ_REQUIRE(M >= 0 && N >= 0 && K > 0 && K % 64 == 0, RDQ_E_INVALID, "rdq_gemm_workspace_size: bad shape M=%d N=%d K=%d", M, N, K);
  *bytes = (M == 0 || N == 0) ? 0 : gemm_workspace_bytes(M, N, K);
  return RDQ_OK;
}

int rdq_quantize_nvfp4(const void *w, int w_is_f32, int n, int K, void *codes, void *scales, float *row_sqerr,
                       float *max_scale, void *stream) {
  RDQ_REQUIRE(n >= 0 && K > 0 && K % 16 == 0, RDQ_E_INVALID, "rdq_quantize_nvfp4 needs n >= 0 and K a positive multiple of 16 (n=%d K=%d)", n, K);
  if (n == 0) return RDQ_OK;
  RDQ_REQUIRE(w != nullptr && codes != nullptr && scales != nullptr, RDQ_E_INVALID, "w, codes and scales must not be null");
  RDQ_REQUIRE(aligned16(w) && (reinterpret_cast<uintptr_t>(codes) & 7) == 0, RDQ_E_INVALID,
              "w must be 16-byte aligned and codes 8-byte aligned");
  return launch_quantize_nvfp4(w, w_is_f32 != 0, n, K, static_cast<uint8_t *>(codes), static_cast<uint8_t *>(scales), row_sqerr,
                               max_scale, static_cast<cudaStream_t>(stream));
}

int rdq_quantize_fp8(const void *w, int w_is_f32, int n, int K, void *out, float *scale_out, float *row_sqerr,
                     float *absmax_scratch, void *stream) {
  RDQ_REQUIRE(n >= 0 && K > 0 && K % 16 == 0, RDQ_E_INVALID, "rdq_quantize_fp8 needs n >= 0 and K a positive multiple of 16 (n=%d K=%d)", n, K);
  if (n == 0) return RDQ_OK;
  RDQ_REQUIRE(w != nullptr && out != nullptr && absmax_scratch != nullptr, RDQ_E_INVALID, "w, out and absmax_scratch must not be null");
  RDQ_REQUIRE(aligned16(w) && aligned16(out), RDQ_E_INVALID, "w and out must be 16-byte aligned");
  return launch_quantize_fp8(w, w_is_f32 != 0, n, K, static_cast<uint8_t *>(out), scale_out, row_sqerr, absmax_scratch,
                             static_cast<cudaStream_t>(stream));
}

int rdq_add_rmsnorm(void *x, const void *delta, const void *weight, void *out, int B, int H, float eps, int flags,
                    void *stream) {
  RDQ_REQUIRE(B >= 0 && H > 0 && H % 8 == 0, RDQ_E_INVALID, "rdq_add_rmsnorm needs H a positive multiple of 8 (B=%d H=%d)", B, H);
  if (B == 0) return RDQ_OK;
  RDQ_REQUIRE(x && weight && out, RDQ_E_INVALID, "x, weight and out must not be null");
  RDQ_REQUIRE(aligned16(x) && aligned16(weight) && aligned16(out) && aligned16(delta), RDQ_E_INVALID,
              "x, delta, weight and out must be 16-byte aligned");
  return launch_add_rmsnorm(static_cast<__half *>(x), static_cast<const __half *>(delta), static_cast<const __half *>(weight),
                            static_cast<__half *>(out), B, H, eps, (flags & RDQ_GEMV_PDL) != 0, static_cast<cudaStream_t>(stream));
}

int rdq_qk_rope_cache(const void *qkv, const void *q_norm, const void *k_norm, const void *cos_table, const void *sin_table,
                      const long long *pos, void *q_out, void *k_cache, void *v_cache, int B, int n_q_heads, int n_kv_heads,
                      int head_dim, int S, float eps, int flags, void *stream) {
  RDQ_REQUIRE(B >= 0 && n_q_heads > 0 && n_kv_heads > 0 && S > 0, RDQ_E_INVALID, "bad attention geometry");
  RDQ_REQUIRE(head_dim >= 64 && head_dim <= 256 && head_dim % 64 == 0, RDQ_E_UNSUPPORTED,
              "head_dim must be 64, 128, 192 or 256, got %d", head_dim);
  if (B == 0) return RDQ_OK;
  RDQ_REQUIRE(qkv && cos_table && sin_table && pos && q_out && k_cache && v_cache, RDQ_E_INVALID, "null pointer");
  return launch_qk_rope_cache(static_cast<const __half *>(qkv), static_cast<const __half *>(q_norm),
                              static_cast<const __half *>(k_norm), static_cast<const __half *>(cos_table),
                              static_cast<const __half *>(sin_table), pos, static_cast<__half *>(q_out),
                              static_cast<__half *>(k_cache), static_cast<__half *>(v_cache), B, n_q_heads, n_kv_heads, head_dim,
                              S, eps, (flags & RDQ_GEMV_PDL) != 0, static_cast<cudaStream_t>(stream));
}

int rdq_attn_decode_scratch_size(int B, int n_q_heads, int head_dim, int S, size_t *bytes) {
  RDQ_REQUIRE(bytes && B >= 0 && n_q_heads > 0 && head_dim > 0 && S > 0, RDQ_E_INVALID, "bad arguments");
  const int nsplit = (S + attn_chunk() - 1) / attn_chunk();
  *bytes = sizeof(float) * static_cast<size_t>(B) * n_q_heads * nsplit * (head_dim + 2);
  return RDQ_OK;
}

int rdq_attn_decode(const void *q, const void *k_cache, const void *v_cache, const long long *pos, void *scratch, void *out,
                    int B, int n_q_heads, int n_kv_heads, int head_dim, int S, float scale, int flags, void *stream) {
  RDQ_REQUIRE(B >= 0 && n_q_heads > 0 && n_kv_heads > 0 && n_q_heads % n_kv_heads == 0 && S > 0, RDQ_E_INVALID,
              "bad attention geometry");
  RDQ_REQUIRE(head_dim >= 32 && head_dim <= 256 && head_dim % 32 == 0, RDQ_E_UNSUPPORTED,
              "head_dim must be a multiple of 32 up to 256, got %d", head_dim);
  if (B == 0) return RDQ_OK;
  RDQ_REQUIRE(q && k_cache && v_cache && pos && scratch && out, RDQ_E_INVALID, "null pointer");
  RDQ_REQUIRE((reinterpret_cast<uintptr_t>(k_cache) & 7) == 0 && (reinterpret_cast<uintptr_t>(v_cache) & 7) == 0, RDQ_E_INVALID,
              "caches must be 8-byte aligned");
  return launch_attn_decode(static_cast<const __half *>(q), static_cast<const __half *>(k_cache),
                            static_cast<const __half *>(v_cache), pos, static_cast<float *>(scratch), static_cast<__half *>(out),
                            B, n_q_heads, n_kv_heads, head_dim, S, scale, (flags & RDQ_GEMV_PDL) != 0,
                            static_cast<cudaStream_t>(stream));
}

int rdq_rope_attn_decode_scratch_size(int B, int n_q_heads, int n_kv_heads, int head_dim, int S, size_t *bytes) {
  RDQ_REQUIRE(bytes && B >= 0 && n_q_heads > 0 && n_kv_heads > 0 && head_dim > 0 && S > 0, RDQ_E_INVALID, "bad arguments");
  *bytes = rope_attn_scratch_bytes(std::max(B, 1), n_q_heads, n_kv_heads, head_dim, S);
  return RDQ_OK;
}

int rdq_rope_attn_decode(const void *qkv, const void *q_norm, const void *k_norm, const void *cos_table, const void *sin_table,
                         const long long *pos, void *k_cache, void *v_cache, void *scratch, void *out, int B, int n_q_heads,
                         int n_kv_heads, int head_dim, int S, float scale, float eps, int flags, void *stream) {
  RDQ_REQUIRE(B >= 0 && n_q_heads > 0 && n_kv_heads > 0 && n_q_heads % n_kv_heads == 0 && S > 0, RDQ_E_INVALID,
              "bad attention geometry");
  RDQ_REQUIRE(head_dim == 64 || head_dim == 128 || head_dim == 256, RDQ_E_UNSUPPORTED,
              "head_dim must be 64, 128 or 256, got %d", head_dim);
  RDQ_REQUIRE(n_q_heads / n_kv_heads <= 16, RDQ_E_UNSUPPORTED, "at most 16 query heads per KV head, got %d",
              n_q_heads / n_kv_heads);
  if (B == 0) return RDQ_OK;
  RDQ_REQUIRE(qkv && cos_table && sin_table && pos && k_cache && v_cache && scratch && out, RDQ_E_INVALID, "null pointer");
  RDQ_REQUIRE(aligned16(k_cache) && aligned16(v_cache) && aligned16(scratch), RDQ_E_INVALID,
              "caches and scratch must be 16-byte aligned");
  return launch_rope_attn(static_cast<const __half *>(qkv), static_cast<const __half *>(q_norm),
                          static_cast<const __half *>(k_norm), static_cast<const __half *>(cos_table),
                          static_cast<const __half *>(sin_table), pos, static_cast<__half *>(k_cache),
                          static_cast<__half *>(v_cache), scratch, static_cast<__half *>(out), B, n_q_heads, n_kv_heads, head_dim,
                          S, scale, eps, (flags & RDQ_GEMV_PDL) != 0, static_cast<cudaStream_t>(stream));
}

int rdq_silu_mul(const void *gate_up, void *out, int B, int F, int flags, void *stream) {
  RDQ_REQUIRE(B >= 0 && F > 0 && F % 8 == 0, RDQ_E_INVALID, "rdq_silu_mul needs F a positive multiple of 8 (B=%d F=%d)", B, F);
  if (B == 0) return RDQ_OK;
  RDQ_REQUIRE(gate_up && out && aligned16(gate_up) && aligned16(out), RDQ_E_INVALID, "gate_up and out must be 16-byte aligned");
  return launch_silu_mul(static_cast<const __half *>(gate_up), static_cast<__half *>(out), B, F, (flags & RDQ_GEMV_PDL) != 0,
                         static_cast<cudaStream_t>(stream));
}

int rdq_stage_copy(void *dst, const void *src, size_t bytes, void *stream) {
  RDQ_REQUIRE(bytes == 0 || (dst != nullptr && src != nullptr), RDQ_E_INVALID, "dst and src must not be null");
  RDQ_REQUIRE(aligned16(dst) && aligned16(src), RDQ_E_INVALID, "dst and src must be 16-byte aligned");
  return launch_stage_copy(dst, src, bytes, nullptr, nullptr, static_cast<cudaStream_t>(stream));
}

int rdq_stage_copy_signal(void *dst, const void *src, size_t bytes, int32_t *state, int32_t *flag, void *stream) {
  RDQ_REQUIRE(bytes == 0 || (dst != nullptr && src != nullptr), RDQ_E_INVALID, "dst and src must not be null");
  RDQ_REQUIRE(aligned16(dst) && aligned16(src), RDQ_E_INVALID, "dst and src must be 16-byte aligned");
  RDQ_REQUIRE(state != nullptr && flag != nullptr, RDQ_E_INVALID, "state and flag must not be null");
  return launch_stage_copy(dst, src, bytes, state, flag, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
